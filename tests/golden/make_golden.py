"""Regenerates tests/golden/*.npz from the CPU oracle.

The reference cannot run here (Rust, no toolchain) and holds no model-level golden vectors for this path, so
these fixtures are the oracle's own outputs on seeded inputs.  They pin the oracle against silent drift and
give the GPU tests a fixed target that does not depend on rebuilding the oracle on the GPU box.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from __graft_entry__ import load_package  # noqa: E402
from oracle import OracleModel  # noqa: E402

CASES = {
    # name: (config, seed, prompt tokens, greedy steps)
    "tiny_f32": ("tiny_f32", 1234, 16, 16),            # the reference's CPU-runnable case: 16-token prompt, 16 steps
    "small_q8": ("small_q8", 99, 12, 24),
}


def main():
    pkg = load_package()
    for name, (cfg, seed, n_prompt, n_new) in CASES.items():
        m = OracleModel(pkg.CONFIGS[cfg])
        m.synth(seed)
        prompt = m.synth_tokens(seed, n_prompt)
        toks, logits, margins = m.generate(prompt, n_new, return_last_logits=True, return_margins=True)
        k0 = m.kv_read(0, "k", n_prompt + n_new - 1)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), config=cfg, seed=seed, prompt=np.array(prompt, dtype=np.int32),
                            tokens=np.array(toks, dtype=np.int32), last_logits=logits.astype(np.float32),
                            margins=np.array(margins, dtype=np.float32), k_cache_layer0=k0.astype(np.float32))
        print(name, "tokens", toks, "min margin", float(min(margins)))


if __name__ == "__main__":
    main()
