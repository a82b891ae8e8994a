"""Host-side plans for running the forward path on several GPUs (one process per GPU).

Two ways to use N GPUs:

* request sharding (``shard_requests``): every rank holds a full replica and serves its own
  requests; there is no data-path collective, throughput adds up;
* tensor parallelism (``tp_plan``): one model is cut over the ranks the way
  ``forge_model_create`` cuts it when ``tp_world > 1``: q/k/v and gate/up keep whole output
  rows (attention heads / FFN channels) per rank, the attention-output and FFN-down projections
  keep a slice of their input dimension, and their partial results are summed over the ranks.

These functions are pure host logic; the tests run them on CPU ranks (gloo).
"""
from __future__ import annotations

from dataclasses import dataclass


def shard_requests(n_requests: int, rank: int, world: int) -> range:
    """Requests served by ``rank``: a contiguous, near-equal share (earlier ranks get the remainder)."""
    if world < 1 or not 0 <= rank < world or n_requests < 0:
        raise ValueError("bad rank/world/request count")
    base, extra = divmod(n_requests, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


@dataclass(frozen=True)
class TpPlan:
    """Slices kept by one rank.  Row ranges are output rows; block ranges are 32-column blocks of the input."""
    q_rows: range
    kv_rows: range          # the same range for k and for v
    ffn_rows: range         # the same range for gate and for up
    o_blocks: range         # input blocks of the attention-output projection (= this rank's q columns / 32)
    down_blocks: range      # input blocks of the FFN-down projection (= this rank's FFN channels / 32)
    num_heads: int
    num_kv_heads: int


def tp_plan(cfg: dict, rank: int, world: int) -> TpPlan:
    """The cut ``forge_model_create`` makes for ``tp_rank = rank`` of ``tp_world = world``."""
    nh, nkv, hd, ff = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"], cfg["intermediate_size"]
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    if nh % world or nkv % world or ff % world or (nh // world * hd) % 32 or (ff // world) % 32:
        raise ValueError("heads, KV heads and FFN channels must divide evenly over the ranks (in whole 32-column blocks)")
    qk, kv, f = nh // world * hd, nkv // world * hd, ff // world
    return TpPlan(range(rank * qk, (rank + 1) * qk), range(rank * kv, (rank + 1) * kv), range(rank * f, (rank + 1) * f),
                  range(rank * qk // 32, (rank + 1) * qk // 32), range(rank * f // 32, (rank + 1) * f // 32),
                  nh // world, nkv // world)


class PeerTimeout(RuntimeError):
    """A rank did not contribute to a host-side exchange within the limit."""


def gather_exchange_handles(mine, world: int, timeout_s: float = 60.0):
    """All ranks' exchange-buffer handles, in rank order (what ``forge_model_tp_exchange_attach`` takes).

    The handles travel over a gloo group created for this one exchange with ``timeout_s`` as its limit: if a
    rank never posts its handle (it died, or never reached this point) the others get ``PeerTimeout`` instead of
    waiting for ever, and nothing has touched a GPU yet.  Needs an initialised ``torch.distributed``.
    """
    import datetime

    import numpy as np
    import torch
    import torch.distributed as dist

    group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
    local = torch.from_numpy(np.ascontiguousarray(mine, dtype=np.uint8).copy())
    parts = [torch.empty_like(local) for _ in range(world)]
    try:
        dist.all_gather(parts, local, group=group)
    except RuntimeError as e:  # gloo reports a missing peer as a timed-out / failed collective
        raise PeerTimeout(f"a rank did not post its exchange handle within {timeout_s} s: {e}") from e
    return torch.cat(parts).numpy()

