"""Host-side sharding for tensor parallelism: which part of every weight a rank holds, and the local geometry its
decoder is built with. Column-parallel projections (wq, wk, wv, gate, up) split the ROWS of the reference's [N, K]
weights; row-parallel ones (wo, down) split K, i.e. a range of whole blocks of every packed row (quantized rows are
sequences of 32- or 256-value blocks: crates/runtime-cpu/src/quantized.rs:263-292). Embedding and norms are replicated; the head is
replicated or, with shard_head, cut by rows (vocabulary parallel: every rank scores vocab / world tokens and the ranks
exchange their best).

Works on numpy arrays and on torch tensors alike (only slicing, reshape and contiguity are used).
"""
from __future__ import annotations

# codec -> (values, bytes) of one block; 0 = dense f32. Q4_0 / Q8_0 blocks hold 32 values, the K-quants 256
# (crates/runtime/src/gguf.rs:245-291).
BLOCKS = {2: (32, 18), 8: (32, 34), 10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210)}
ROW_SPLIT = ("wq", "wk", "wv", "gate", "up")
COLUMN_SPLIT = ("wo", "down")


def check_geometry(cfg: dict, world: int) -> None:
    """Raises ValueError when the model cannot be cut into `world` shards."""
    if world < 1:
        raise ValueError("world size must be positive")
    for key in ("q_heads", "kv_heads", "ffn"):
        if cfg[key] % world:
            raise ValueError(f"{key} = {cfg[key]} is not divisible by the {world} ranks")
    if (cfg["ffn"] // world) % 64 or (cfg["q_heads"] // world * cfg["head_dim"]) % 64:
        raise ValueError("a rank's share of ffn and of q_heads * head_dim must be a multiple of 64 columns")


def local_config(cfg: dict, world: int, shard_head: bool = False, rank: int = 0) -> dict:
    """The geometry one rank's decoder and KV pool are created with. shard_head: `vocab` becomes this rank's number of
    head rows and `vocab_global` / `head_first_row` say where they sit (Executable takes both)."""
    check_geometry(cfg, world)
    out = dict(cfg)
    out["q_heads"] = cfg["q_heads"] // world
    out["kv_heads"] = cfg["kv_heads"] // world
    out["ffn"] = cfg["ffn"] // world
    if shard_head and world > 1:
        if cfg["vocab"] % world:
            raise ValueError(f"vocab = {cfg['vocab']} is not divisible by the {world} ranks")
        out["vocab"] = cfg["vocab"] // world
        out["vocab_global"] = cfg["vocab"]
        out["head_first_row"] = rank * out["vocab"]
    return out


def _contiguous(x):
    return x.contiguous() if hasattr(x, "contiguous") else __import__("numpy").ascontiguousarray(x)


def shard_rows(weight, rank: int, world: int):
    """Rows [rank * N / world, (rank + 1) * N / world) of a dense or packed [N, ...] matrix."""
    n = weight.shape[0]
    if n % world:
        raise ValueError(f"{n} rows are not divisible by {world}")
    per = n // world
    return _contiguous(weight[rank * per:(rank + 1) * per])


def shard_columns(weight, codec: int, rank: int, world: int):
    """Columns [rank * K / world, (rank + 1) * K / world) of every row: f32 elements, or whole blocks of the codec."""
    if codec != 0 and codec not in BLOCKS:
        raise ValueError(f"unknown block codec {codec}")
    unit = 1 if codec == 0 else BLOCKS[codec][1]
    width = weight.shape[1]
    if width % unit:
        raise ValueError("row width is not a whole number of blocks")
    units = width // unit
    granule = 32 if codec == 0 else 1  # a dense shard keeps 32-column alignment like a packed one
    if units % (world * granule):
        raise ValueError(f"{units} column units are not divisible by {world} ranks")
    per = units // world * unit
    return _contiguous(weight[:, rank * per:(rank + 1) * per])


def shard_weights(weights: dict, cfg: dict, rank: int, world: int, shard_head: bool = False) -> dict:
    """One rank's share of a weight dictionary laid out like tests/helpers.make_weights: projections are either dense
    [N, K] arrays or (packed, rows, columns[, codec]) tuples."""
    check_geometry(cfg, world)
    codec = weights["codec"]

    def rows(value):
        if isinstance(value, tuple):
            packed, n, k = value[:3]
            return (shard_rows(packed, rank, world), n // world, k) + tuple(value[3:])
        return shard_rows(value, rank, world)

    def columns(value):
        if isinstance(value, tuple):  # (packed, rows, columns) of the dictionary's codec, or with a codec of its own as 4th entry
            packed, n, k = value[:3]
            own = value[3] if len(value) > 3 else codec
            return (shard_columns(packed, own, rank, world), n, k // world) + tuple(value[3:])
        return shard_columns(value, 0, rank, world)

    head = rows(weights["head"]) if shard_head and world > 1 else weights["head"]
    out = {"tok_embd": weights["tok_embd"], "out_norm": weights["out_norm"], "head": head, "codec": codec, "layers": []}
    for layer in weights["layers"]:
        local = dict(layer)
        for name in ROW_SPLIT:
            local[name] = rows(layer[name])
        for name in COLUMN_SPLIT:
            local[name] = columns(layer[name])
        out["layers"].append(local)
    return out


def all_ranks_ok(ok: bool, group=None) -> bool:
    """Step-status exchange over the host transport (a torch.distributed group, gloo or nccl-backed): True only when
    every rank's step succeeded. A rank observes only its own device status word, so a step in which one rank's bounded
    wait ran out (or any other rank-local failure) is reported as ETC_OK on the others; every rank calls this after
    each tensor-parallel step and treats the step as failed when it returns False."""
    import torch
    import torch.distributed as dist

    flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
    backend = dist.get_backend(group)
    if backend == "nccl":
        flag = flag.cuda()
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(int(flag.item()))


def barrier_before_teardown(group=None) -> None:
    """Host barrier every rank passes before destroying a decoder whose exchange region its peers have mapped: a peer
    may still be reading this rank's partial sums until its own step has been synchronised."""
    import torch.distributed as dist

    dist.barrier(group=group)
