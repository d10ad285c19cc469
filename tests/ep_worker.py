"""One rank of the expert-parallel GPU test (launched under torchrun by tests/test_gpu_ep.py).  Every rank decodes its OWN
sequence; the experts are spread over the ranks and each layer's tokens travel to them and back all-to-all.  Each rank then
compares its tokens and logits with the same model held whole on its own GPU."""
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
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_package()
    from oneiron_luminal_b200 import tp as T
    desc = pkg.CONFIGS[cfg_name]
    T.validate_ep(desc, world)
    uid = T.exchange_unique_id(dist, rank, pkg.B200Runtime.tp_unique_id, device=torch.device("cuda", local))
    rt = pkg.B200Runtime.initialize(device=local)
    rt.tp_init(uid, world, rank)
    rt.load_model(desc.copy(ep_size=world, ep_rank=rank))
    rt.synth(seed)
    prompt = [(7 * i + 3 + 11 * rank) % desc.vocab for i in range(10)]       # a different sequence on every rank, the same length
    toks = rt.generate(prompt, n_new)
    logits = rt.get_f32()
    rt.close()
    ref = pkg.B200Runtime.initialize(device=local)
    ref.load_model(desc)
    ref.synth(seed)
    want = ref.generate(prompt, n_new)
    want_logits = ref.get_f32()
    ref.close()
    err = float(np.max(np.abs(logits - want_logits)) / np.max(np.abs(want_logits)))
    ok = torch.tensor([1 if (toks == want and err <= 1e-3) else 0], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    assert toks == want, (rank, toks, want)
    assert err <= 1e-3, (rank, err)
    if rank == 0 and int(ok.item()) == 1:
        print(f"EP{world} OK tokens={toks[:6]}... logits_rel_err={err:.2e}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
