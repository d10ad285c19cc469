"""One rank of the tensor-parallel GPU test (launched under torchrun by tests/test_gpu_tp.py).  Every rank runs the
sharded model; rank 0 also runs the same model unsharded on its GPU and compares tokens and logits."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from __graft_entry__ import load_package  # noqa: E402


def main():
    cfg_name, seed, n_new = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    n_prompt = int(sys.argv[4]) if len(sys.argv) > 4 else 12
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_package()
    from oneiron_luminal_b200 import tp as T
    desc = pkg.CONFIGS[cfg_name]
    T.validate(desc, world)
    uid = T.exchange_unique_id(dist, rank, pkg.B200Runtime.tp_unique_id, device=torch.device("cuda", local))
    rt = pkg.B200Runtime.initialize(device=local)
    rt.tp_init(uid, world, rank)
    rt.load_model(desc.copy(tp_size=world, tp_rank=rank))
    if os.environ.get("LUM_TP_FUSED", "1") != "0":
        # exchange of partial sums through peer memory (no collective kernel between the projections)
        rt.tp_peer_import(T.exchange_peer_handles(dist, world, rt.tp_peer_export(), device=torch.device("cuda", local)))
    rt.synth(seed)
    prompt = [(7 * i + 3) % desc.vocab for i in range(n_prompt)]
    if os.environ.get("LUM_TP_SAMPLE", "0") == "1":
        sampled_run(rt, desc, prompt, n_new, rank, world)
        rt.close()
        dist.barrier()
        dist.destroy_process_group()
        return
    toks = rt.generate(prompt, n_new)
    logits = rt.get_f32()                       # this rank's vocabulary shard
    shard = desc.vocab // world
    gathered = [torch.zeros(shard, device="cuda") for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(logits).cuda())
    full = torch.cat(gathered).cpu().numpy()
    tok_t = torch.tensor(toks, device="cuda")
    all_toks = [torch.zeros_like(tok_t) for _ in range(world)]
    dist.all_gather(all_toks, tok_t)
    assert all((t == tok_t).all().item() for t in all_toks), "ranks disagree on the sampled tokens"
    rt.close()
    if rank == 0:
        ref = pkg.B200Runtime.initialize(device=local, prefill_min_rows=1 << 30)      # same per-token prompt path as the sharded ranks
        ref.load_model(desc)
        ref.synth(seed)
        want = ref.generate(prompt, n_new)
        want_logits = ref.get_f32()
        ref.close()
        err = float(np.max(np.abs(full - want_logits)) / np.max(np.abs(want_logits)))
        assert toks == want, (toks, want)
        assert err <= 1e-3, err
        print(f"TP{world} OK tokens={toks[:6]}... logits_rel_err={err:.2e}")
    dist.barrier()
    dist.destroy_process_group()


def sampled_run(rt, desc, prompt, n_new, rank, world):
    """With a sampler set: every step's draw equals the oracle's draw from the gathered logits of that step, every rank draws the
    same tokens, and the device-resident loop replays the token-by-token run."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    T_, K_, P_, S_ = 0.8, 40, 0.9, 4242
    rt.set_sampling(T_, K_, P_, S_)
    shard = desc.vocab // world

    def gathered_logits():
        parts = [torch.zeros(shard, device="cuda") for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(rt.get_f32()).cuda())
        return torch.cat(parts).cpu().numpy()

    rt.kv_reset(); rt.decode_reset()
    rt.set_data(prompt); rt.execute({"s": len(prompt), "p": 0})
    toks, pos, near = [], len(prompt), 0
    for _ in range(n_new):
        tok = rt.get_token()
        want, margin = oracle.sample_topk(gathered_logits(), T_, K_, P_, S_, 0, pos)
        if margin >= 1e-5:
            assert tok == want, (rank, len(toks), tok, want, margin)
        else:
            near += 1
        toks.append(tok)
        rt.set_data([tok]); rt.execute({"s": 1, "p": pos})
        pos += 1
    assert near <= 1
    tok_t = torch.tensor(toks, device="cuda")
    all_toks = [torch.zeros_like(tok_t) for _ in range(world)]
    dist.all_gather(all_toks, tok_t)
    assert all((t == tok_t).all().item() for t in all_toks), "ranks disagree on the drawn tokens"
    again = rt.generate(prompt, n_new)
    assert again == toks, (again, toks)
    if rank == 0:
        print(f"TP{world} OK sampled tokens={toks[:6]}...")


if __name__ == "__main__":
    main()
