"""Multi-rank host logic on CPU ranks (gloo, world size 2): request sharding and the tensor-parallel cut.

The tensor-parallel case plays one attention + FFN projection chain with the CPU restatement of the quantised
matmul: every rank works on the slices `tp_plan` gives it, row-sliced partial products are summed with an
all-reduce, and the result must match the uncut computation."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from forge_llm_b200 import configs, parallel, synth  # noqa: E402


def test_shard_requests_partitions():
    for n in (0, 1, 7, 8, 129):
        for world in (1, 2, 3, 8):
            got = [i for r in range(world) for i in parallel.shard_requests(n, r, world)]
            assert got == list(range(n))
            sizes = [len(parallel.shard_requests(n, r, world)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.shard_requests(4, 2, 2)


def test_tp_plan_covers_every_row_once():
    c = configs.CONFIGS["c5"]
    for world in (1, 2, 4):
        plans = [parallel.tp_plan(c, r, world) for r in range(world)]
        assert [i for p in plans for i in p.q_rows] == list(range(c["num_heads"] * c["head_dim"]))
        assert [i for p in plans for i in p.kv_rows] == list(range(c["num_kv_heads"] * c["head_dim"]))
        assert [i for p in plans for i in p.ffn_rows] == list(range(c["intermediate_size"]))
        assert [i for p in plans for i in p.down_blocks] == list(range(c["intermediate_size"] // 32))
        assert sum(p.num_heads for p in plans) == c["num_heads"]
    with pytest.raises(ValueError):
        parallel.tp_plan(configs.CONFIGS["c1"], 0, 4)  # 9 heads do not divide over 4 ranks


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, quant: int):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from oracle import oracle
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        c = configs.tiny(quant=quant, hd=64, nq=4, nkv=2, hidden=256, ffn=512)
        H, QK, FF = c["hidden_size"], c["num_heads"] * c["head_dim"], c["intermediate_size"]
        BS = 34 if quant == 8 else 18
        rng = np.random.default_rng(5)  # the same stream on every rank
        wq = synth.quantize(quant, rng.standard_normal((QK, H), dtype=np.float32) * 0.05).reshape(QK, H // 32, BS)
        wo = synth.quantize(quant, rng.standard_normal((H, QK), dtype=np.float32) * 0.05).reshape(H, QK // 32, BS)
        wg = synth.quantize(quant, rng.standard_normal((FF, H), dtype=np.float32) * 0.05).reshape(FF, H // 32, BS)
        wd = synth.quantize(quant, rng.standard_normal((H, FF), dtype=np.float32) * 0.05).reshape(H, FF // 32, BS)
        x = rng.standard_normal((3, H), dtype=np.float32)
        plan = parallel.tp_plan(c, rank, world)

        def mm(a, w):  # w: [N][K/32][BS]
            return oracle.matmul_mat(quant, np.ascontiguousarray(a), np.ascontiguousarray(w).reshape(-1), w.shape[1] * 32, w.shape[0])

        def col_sliced(a, w, rows):  # every rank computes its own output rows; gathered = the full product
            mine = torch.from_numpy(mm(a, w[rows.start:rows.stop]))
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            return mine.numpy(), torch.cat(parts, dim=1).numpy()

        def row_sliced(a_local, w, blocks):  # partial products over this rank's input blocks, summed over the ranks
            part = torch.from_numpy(mm(a_local, w[:, blocks.start:blocks.stop]))
            dist.all_reduce(part, op=dist.ReduceOp.SUM)
            return part.numpy()

        q_mine, q_all = col_sliced(x, wq, plan.q_rows)
        assert np.array_equal(q_all, mm(x, wq))                      # rows are computed exactly as in the uncut product
        o = row_sliced(q_mine, wo, plan.o_blocks)                    # (attention left out: the cut is what is tested)
        o_ref = mm(mm(x, wq), wo)
        assert np.linalg.norm(o - o_ref) / np.linalg.norm(o_ref) < 1e-6
        g_mine, g_all = col_sliced(x, wg, plan.ffn_rows)
        assert np.array_equal(g_all, mm(x, wg))
        d = row_sliced(g_mine, wd, plan.down_blocks)
        d_ref = mm(mm(x, wg), wd)
        assert np.linalg.norm(d - d_ref) / np.linalg.norm(d_ref) < 1e-6
        # request sharding: the aggregate of per-rank counts is the job (the bench's reduction)
        mine = torch.tensor([float(len(parallel.shard_requests(11, rank, world)))])
        dist.all_reduce(mine, op=dist.ReduceOp.SUM)
        assert mine.item() == 11.0
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("quant", [8, 4])
def test_tensor_parallel_cut_on_two_cpu_ranks(quant, oracle):
    import torch.multiprocessing as mp
    mp.spawn(_rank_main, args=(2, _free_port(), quant), nprocs=2, join=True)


def _handle_rank(rank: int, world: int, port: int, posts: bool, out):
    import datetime
    import time

    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=30))
    mine = np.full(64, rank + 1, np.uint8)
    try:
        if rank == 1 and not posts:
            # this rank joins the group (group creation is collective) but never contributes its handle
            import torch
            dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=1.5))
            time.sleep(4.0)
            out.put((rank, "silent"))
            return
        try:
            got = parallel.gather_exchange_handles(mine, world, timeout_s=1.5)
            out.put((rank, got.tolist()))
        except parallel.PeerTimeout:
            out.put((rank, "timeout"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("posts", [True, False])
def test_exchange_handles_gather_and_silent_rank(posts):
    """Every rank gets all handles in rank order; a rank that never posts makes the others fail with PeerTimeout
    within the limit instead of waiting (the failure is made on the host: no GPU is involved)."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_handle_rank, args=(r, 2, port, posts, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(out.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    if posts:
        want = [1] * 64 + [2] * 64
        assert got[0] == want and got[1] == want
    else:
        assert got[0] == "timeout" and got[1] == "silent"

