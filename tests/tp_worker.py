"""One rank of the tensor-parallel parity check on GPUs; tests/test_gpu_tensor_parallel.py launches world_size of these
with torch.distributed.run. Every rank builds its shard of a small Q4_0 model; rank 0 also runs the CPU oracle on the
whole model. Checked: teacher-forced logits against the oracle (2e-3), identical tokens on all ranks, and the
device-resident greedy loop (CUDA graph with the all-reduces captured) against step-by-step execution: with the NCCL
all-reduce, with the peer-memory all-reduce (one shot by default at these sizes, reduce-scatter + all-gather forced), and with a vocabulary-parallel head whose ranks exchange their best logit."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import effect_torch_b200 as et  # noqa: E402
import oracle as orc  # noqa: E402
from effect_torch_b200 import tensor_parallel as tp  # noqa: E402
from tests import helpers  # noqa: E402

LOGIT_TOL = 2e-3


def build(rt, cfg, weights, batch, max_tokens):
    dec = et.Executable(rt, layers=cfg["layers"], d_model=cfg["d_model"], q_heads=cfg["q_heads"], kv_heads=cfg["kv_heads"],
                        head_dim=cfg["head_dim"], ffn=cfg["ffn"], vocab=cfg["vocab"], rms_eps=cfg["rms_eps"],
                        rope_theta=cfg["rope_theta"], batch=batch, max_tokens=max_tokens, block_size=16, kv_dtype=et.KV_F16,
                        exact=False, max_advance=8, vocab_global=cfg.get("vocab_global"), head_first_row=cfg.get("head_first_row", 0))
    helpers.load_into(dec, weights)
    dec.finalize()
    return dec


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    cfg = dict(helpers.TINY_Q, q_heads=8, kv_heads=4, head_dim=64, d_model=512) if world > 2 else helpers.TINY_Q
    weights = helpers.make_weights(cfg, seed=3, codec=orc.Q4_0)  # the same seed everywhere: replicated host state
    B, max_tokens = 3, 512
    rt = et.Runtime(local)
    lcfg = tp.local_config(cfg, world)
    replicated = dec = build(rt, lcfg, tp.shard_weights(weights, cfg, rank, world), B, max_tokens)
    ident = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        ident = torch.frombuffer(bytearray(et.tensor_parallel_id()), dtype=torch.uint8).clone()
    dist.broadcast(ident, src=0)
    dec.set_tensor_parallel(rank, world, bytes(ident.tolist()))
    pool = et.NativeKvPool(rt, lcfg["layers"], lcfg["kv_heads"], lcfg["head_dim"], max_tokens, 16, et.KV_F16)
    failures = []
    odec = helpers.oracle_decoder(cfg, weights, batch=B) if rank == 0 else None

    def same_on_all_ranks(array):
        mine = torch.from_numpy(np.ascontiguousarray(array).copy())
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        return all(torch.equal(everyone[0], e) for e in everyone[1:])

    def run_checks(tag, dec=None, sharded_head=False):
        dec = dec or replicated
        seqs = [pool.makeSequence() for _ in range(B)]
        if rank == 0:
            opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], max_tokens, 16, orc.F16)
            oseqs = [opool.make_sequence() for _ in range(B)]
        rng = np.random.default_rng(2)
        for advance in (8, 5, 1, 1, 1):
            toks = rng.integers(0, cfg["vocab"], size=(B, advance)).astype(np.uint32)
            gl = dec.execute(pool, seqs, toks)
            if sharded_head:  # every rank returns its slice of the vocabulary: put the slices side by side
                mine = torch.from_numpy(gl.copy())
                slices = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(slices, mine)
                gl = torch.cat(slices, dim=1).numpy()
            if rank == 0:
                ol, _ = odec.execute(opool, oseqs, toks)
                err = helpers.rel_err(gl, ol)
                if err > LOGIT_TOL:
                    failures.append(f"{tag}: advance {advance}: logits rel err {err:.3e}")
            if not same_on_all_ranks(gl):
                failures.append(f"{tag}: advance {advance}: ranks hold different logits")
        for s in seqs:
            s.release()
        # step by step, then the same continuation device-resident on a second set of sequences
        first = rng.integers(0, cfg["vocab"], size=B).astype(np.uint32)
        prompt = rng.integers(0, cfg["vocab"], size=(B, 8)).astype(np.uint32)
        outs = []
        for mode in ("stepwise", "resident"):
            s2 = [pool.makeSequence() for _ in range(B)]
            dec.execute(pool, s2, prompt)
            if mode == "stepwise":
                tok, out = first, []
                for _ in range(12):
                    tok = dec.executeSampled(pool, s2, tok[:, None])
                    out.append(tok)
                outs.append(np.stack(out))
            else:
                out, _ = dec.generate_greedy(pool, s2, first, 12)
                outs.append(out)
            for s in s2:
                s.release()
        if not np.array_equal(outs[0], outs[1]):
            failures.append(f"{tag}: device-resident generation differs from step-by-step execution")
        if not same_on_all_ranks(outs[1].astype(np.int64)):
            failures.append(f"{tag}: ranks generated different tokens")
        return outs[1]

    tokens_nccl = run_checks("nccl all-reduce")
    # the same again with the one-shot all-reduce over peer memory
    mine = torch.frombuffer(bytearray(dec.peer_exchange_handle()), dtype=torch.uint8).clone()
    table = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(table, mine)
    dec.use_peer_allreduce([bytes(t.tolist()) for t in table])
    tokens_peer = run_checks("peer-memory all-reduce")
    del tokens_nccl  # NCCL adds in its own order: equal within the logits tolerance checked above, not bit for bit

    def second_decoder(tag, shard_head, two_shot):
        """A decoder of its own (the exchange regions are per decoder) with the given head layout and all-reduce kind."""
        os.environ["ETC_TP_TWO_SHOT"] = "1" if two_shot else "0"
        cfg2 = tp.local_config(cfg, world, shard_head=shard_head, rank=rank)
        dec2 = build(rt, cfg2, tp.shard_weights(weights, cfg, rank, world, shard_head=shard_head), B, max_tokens)
        ident2 = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            ident2 = torch.frombuffer(bytearray(et.tensor_parallel_id()), dtype=torch.uint8).clone()
        dist.broadcast(ident2, src=0)
        dec2.set_tensor_parallel(rank, world, bytes(ident2.tolist()))
        mine = torch.frombuffer(bytearray(dec2.peer_exchange_handle()), dtype=torch.uint8).clone()
        table = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(table, mine)
        dec2.use_peer_allreduce([bytes(t.tolist()) for t in table])
        tokens = run_checks(tag, dec2, sharded_head=shard_head)
        dist.barrier()  # nobody reads this decoder's region any more
        dec2.close()
        return tokens

    tokens_other = second_decoder("the other peer all-reduce kind", False, two_shot=True)
    tokens_vocab = second_decoder("vocabulary-parallel head", True, two_shot=world >= 4)
    for name, got in (("the other peer all-reduce kind", tokens_other), ("the vocabulary-parallel head", tokens_vocab)):
        if not np.array_equal(got, tokens_peer):  # one-shot and two-shot add in rank order: the same sums, the same tokens
            failures.append(f"{name} generated different tokens from the default peer path")

    flag = torch.tensor([len(failures)])
    dist.all_reduce(flag)
    for f in failures:
        print(f"[rank {rank}] {f}", flush=True)
    dec.close()
    dist.destroy_process_group()
    if rank == 0 and flag.item() == 0:
        print("tensor parallel parity ok", flush=True)
    sys.exit(1 if flag.item() else 0)


if __name__ == "__main__":
    main()
