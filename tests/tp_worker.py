"""One rank of the tensor-parallel parity check (launched by test_tp_gpu.py under torch.distributed.run).

Every rank builds the same synthetic model with tp_world = WORLD_SIZE on its own GPU; rank 0 compares the
logits of a prefill, of teacher-forced decode steps (single-sequence and batched), and the greedy ids, with the CPU
restatement.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    from forge_llm_b200 import configs, runtime, synth

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")  # host channel only: the data path uses the library's own communicator
    key, layers, vocab, n_prompt, n_new = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5])
    c = configs.reduced(key, layers, vocab)
    blob = synth.make_weights_bin(c)
    toks = synth.prompt_tokens(c, n_prompt)
    uid = torch.from_numpy(runtime.Model.tp_unique_id() if rank == 0 else np.zeros(runtime.TP_ID_BYTES, np.uint8))
    dist.broadcast(uid, 0)
    gm = runtime.Model(c, blob, device=local, tp_rank=rank, tp_world=world)
    gm.tp_init(uid.numpy())
    if len(sys.argv) > 6 and sys.argv[6] == "peer":  # decode sums over peer memory instead of the library all-reduce
        from forge_llm_b200 import parallel
        gm.tp_exchange_attach(parallel.gather_exchange_handles(gm.tp_exchange_handle(), world))
        dist.barrier()
    kv = gm.new_cache(max_seq=n_prompt + n_new + 8)
    lg = gm.forward_prefill(toks, kv)
    steps = [lg]
    ok = True
    if rank == 0:
        from oracle import oracle
        om = oracle.OracleModel(c, blob, kv_mode=oracle.KV_F16)
        lo = om.forward_prefill(toks)
        ref = [lo]
    # teacher-forced decode (rank 0 broadcasts the reference's greedy token)
    for _ in range(3):
        t = torch.tensor([int(oracle.argmax(ref[-1])) if rank == 0 else 0], dtype=torch.int64)
        dist.broadcast(t, 0)
        steps.append(gm.forward(int(t.item()), kv))
        if rank == 0:
            ref.append(om.forward(int(t.item())))
    # every rank ends with identical logits
    mine = torch.from_numpy(np.stack(steps))
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    same = all(torch.equal(g, gathered[0]) for g in gathered)
    # free-running greedy generation
    kv.reset()
    ids = gm.generate_greedy(toks, n_new, kv)
    if rank == 0:
        om.reset()
        ref_ids, _ = om.generate_greedy(toks, n_new)
        worst = max(float(np.abs(a - b).max()) for a, b in zip(steps, ref))
        ok = same and worst < 2e-2 and np.array_equal(ids, ref_ids)
        print(f"TP{world} {key}: ranks identical={same} worst |dlogit|={worst:.3e} greedy ids equal={np.array_equal(ids, ref_ids)}", flush=True)
    # a batched step (four sequences of different lengths): teacher-forced logits of every sequence, three steps
    nb = 4
    kvb = gm.new_cache(max_seq=n_prompt + 16, batch=nb)
    prompts = [synth.prompt_tokens(c, n_prompt - 7 * b, seed=20 + b) for b in range(nb)]
    last, oms = [], []
    for b in range(nb):
        gm.forward_prefill(prompts[b], kvb, seq=b, want_logits=False)
        if rank == 0:
            om_b = oracle.OracleModel(c, blob, kv_mode=oracle.KV_F16)
            last.append(om_b.forward_prefill(prompts[b]))
            oms.append(om_b)
    worst_b, same_b = 0.0, True
    for _ in range(3):
        t = torch.tensor([int(oracle.argmax(l)) for l in last] if rank == 0 else [0] * nb, dtype=torch.int64)
        dist.broadcast(t, 0)
        lgb = gm.forward_batch(t.numpy().astype(np.uint32), kvb)
        mine = torch.from_numpy(np.ascontiguousarray(lgb))
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        same_b = same_b and all(torch.equal(g, gathered[0]) for g in gathered)
        if rank == 0:
            last = [oms[b].forward(int(t[b].item())) for b in range(nb)]
            worst_b = max(worst_b, max(float(np.abs(lgb[b] - last[b]).max()) for b in range(nb)))
    kvb.close()
    if rank == 0:
        ok = ok and same_b and worst_b < 2e-2
        print(f"TP{world} {key} batched step: ranks identical={same_b} worst |dlogit|={worst_b:.3e}", flush=True)
    flag = torch.tensor([1 if ok else 0])
    dist.broadcast(flag, 0)
    kv.close()
    gm.close()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
