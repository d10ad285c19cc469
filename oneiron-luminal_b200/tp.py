"""Host-side plumbing for tensor parallelism: one process per GPU, `torch.distributed` only carries the 128-byte
communicator id and a barrier; all data-path exchange happens inside the C-ABI library (NCCL over NVLink).

The reference is single-GPU (crates/luminal_cuda/src/runtime.rs:123-130), so nothing here replaces a reference
interface; the sharding follows the usual Megatron split of a decoder layer: q/k/v/gate/up by output rows
(whole heads), o/down by input columns, lm_head by vocabulary rows; norms and the embedding replicated.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

ROW_SHARDED = ("q", "k", "v", "gate", "up", "lm_head")
COL_SHARDED = ("o", "down")


def full_shape(desc, slot: str) -> Tuple[int, int]:
    qd, kvd = desc.n_q_heads * desc.head_dim, desc.n_kv_heads * desc.head_dim
    return {
        "q": (qd, desc.hidden), "k": (kvd, desc.hidden), "v": (kvd, desc.hidden), "o": (desc.hidden, qd),
        "gate": (desc.ffn, desc.hidden), "up": (desc.ffn, desc.hidden), "down": (desc.hidden, desc.ffn),
        "lm_head": (desc.vocab, desc.hidden), "embed": (desc.vocab, desc.hidden),
        "attn_norm": (1, desc.hidden), "mlp_norm": (1, desc.hidden), "final_norm": (1, desc.hidden),
        "q_norm": (1, desc.head_dim), "k_norm": (1, desc.head_dim),
    }[slot]


def shard_of(desc, slot: str, tp_size: int, tp_rank: int) -> Dict[str, int]:
    """The sub-matrix of `slot` rank `tp_rank` holds: {row0, rows, col0, cols} in the full tensor."""
    n, k = full_shape(desc, slot)
    if tp_size < 1 or not 0 <= tp_rank < tp_size:
        raise ValueError("bad tensor-parallel rank")
    if slot in ROW_SHARDED:
        if n % tp_size:
            raise ValueError(f"{slot}: {n} rows do not divide by {tp_size}")
        return {"row0": tp_rank * (n // tp_size), "rows": n // tp_size, "col0": 0, "cols": k}
    if slot in COL_SHARDED:
        if k % tp_size:
            raise ValueError(f"{slot}: {k} columns do not divide by {tp_size}")
        return {"row0": 0, "rows": n, "col0": tp_rank * (k // tp_size), "cols": k // tp_size}
    return {"row0": 0, "rows": n, "col0": 0, "cols": k}


def validate(desc, tp_size: int) -> None:
    """Raise if the model cannot be split over `tp_size` ranks (whole KV heads per rank, Q8_0 blocks intact)."""
    if desc.n_kv_heads % tp_size or desc.n_q_heads % tp_size or desc.ffn % tp_size or desc.vocab % tp_size:
        raise ValueError("kv heads, q heads, ffn and vocab must divide by the number of ranks")
    if desc.weight_dtype == 7:
        for slot in COL_SHARDED:
            if shard_of(desc, slot, tp_size, 0)["cols"] % 32:
                raise ValueError(f"{slot}: a K-shard must hold whole 32-element Q8_0 blocks")


def validate_ep(desc, ep_size: int) -> None:
    """Raise if the model's experts cannot be spread over `ep_size` ranks (a mixture-of-experts model, whole experts per rank)."""
    if getattr(desc, "n_experts", 0) <= 0:
        raise ValueError("expert parallelism needs a mixture-of-experts model")
    if ep_size < 1 or desc.n_experts % ep_size:
        raise ValueError(f"{desc.n_experts} experts do not divide over {ep_size} ranks")


def local_experts(desc, ep_size: int, ep_rank: int) -> range:
    """The experts rank `ep_rank` holds: a contiguous block, as lum_model_desc.ep_size / ep_rank lay them out."""
    validate_ep(desc, ep_size)
    if not 0 <= ep_rank < ep_size:
        raise ValueError("bad expert-parallel rank")
    per = desc.n_experts // ep_size
    return range(ep_rank * per, (ep_rank + 1) * per)


def exchange_unique_id(dist, rank: int, make_id: Callable[[], bytes], device=None) -> bytes:
    """Rank 0 makes the 128-byte communicator id; everybody gets it through `torch.distributed` (any backend)."""
    import torch
    buf = torch.zeros(128, dtype=torch.uint8, device=device)
    if rank == 0:
        raw = make_id()
        if len(raw) != 128:
            raise ValueError("communicator id must be 128 bytes")
        buf.copy_(torch.tensor(list(raw), dtype=torch.uint8))
    dist.broadcast(buf, src=0)
    return bytes(buf.cpu().tolist())


def exchange_peer_handles(dist, world: int, handle: bytes, device=None):
    """All-gather the ranks' 64-byte IPC handles (rank order) through `torch.distributed` (any backend)."""
    import torch
    mine = torch.tensor(list(handle), dtype=torch.uint8, device=device)
    out = [torch.zeros(64, dtype=torch.uint8, device=device) for _ in range(world)]
    dist.all_gather(out, mine)
    return [bytes(t.cpu().tolist()) for t in out]
