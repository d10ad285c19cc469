"""Regenerates tests/golden/*.npz from the CPU oracle.

The reference cannot run here (Rust, no toolchain) and holds no model-level golden vectors for this path, so
these fixtures are the oracle's own outputs on seeded inputs.  They pin the oracle against silent drift and
give the GPU tests a fixed target that does not depend on rebuilding the oracle on the GPU box.

    python tests/golden/make_golden.py                 # the small cases (seconds)
    python tests/golden/make_golden.py llama3_8b_q8    # a full-size case (tens of minutes of CPU time, ~12 GB of RAM)
    python tests/golden/make_golden.py qwen3_4b_q8
    python tests/golden/make_golden.py gpt_oss_20b_q8  # ~23 GB of RAM
    python tests/golden/make_golden.py llama3_8b_q8_prefill4096   # a 4096-token prompt: about two and a half hours on 8 cores
    python tests/golden/make_golden.py llama3_8b_q8_batch4        # four sequences for batched decode: about 40 minutes

Full-size cases are the configurations the benchmark numbers are quoted on: whole model, whole vocabulary, the
benchmark's seed and prompt.  They hold the prompt, the first 32 greedy tokens with their top-1/top-2 margins,
the logits row that follows the prompt and the one that produced the 32nd token, and a few K/V cache rows of
the first and the last layer.
"""
import os
import sys
import time

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

# name: (config, seed, prompt tokens, greedy steps); the seed and prompt lengths are bench.py's
FULL_SEED = 20240607
FULL_CASES = {
    "llama3_8b_q8": ("llama3_8b_q8", FULL_SEED, 512, 32),
    "qwen3_4b_q8": ("qwen3_4b_q8", FULL_SEED, 1024, 32),
    # routed experts, sliding-window / full layers alternating, sinks, YaRN: 256 tokens take the window (128) out of reach of the start
    "gpt_oss_20b_q8": ("gpt_oss_20b_q8", FULL_SEED, 256, 32),
    # the tensor-core prompt workload's own size: 4096 rows in one pass, the sample that follows (hours of CPU time)
    "llama3_8b_q8_prefill4096": ("llama3_8b_q8", FULL_SEED, 4096, 1),
}


def full_case(pkg, name):
    cfg, seed, n_prompt, n_new = FULL_CASES[name]
    d = pkg.CONFIGS[cfg].copy(max_seq=n_prompt + n_new + 8)      # the oracle's cache is f32: keep it no larger than needed
    t0 = time.time()
    m = OracleModel(d)
    m.synth(seed)
    prompt = m.synth_tokens(seed, n_prompt)
    print(f"{name}: model ready after {time.time() - t0:.0f} s", flush=True)
    m.kv_reset()
    logits = m.forward(prompt, 0)[0]
    prompt_logits = logits.copy()
    toks, margins = [m.argmax(logits)], [m.margin(logits)]
    print(f"{name}: prompt done after {time.time() - t0:.0f} s", flush=True)
    p = n_prompt
    while len(toks) < n_new:
        logits = m.forward([toks[-1]], p)[0]
        p += 1
        toks.append(m.argmax(logits))
        margins.append(m.margin(logits))
    rows = p                                             # cache rows written: the prompt and the first n_new - 1 tokens
    pick = sorted(i for i in {0, 1, n_prompt // 2 - 1, n_prompt - 1, n_prompt, rows - 1} if i < rows)
    L = d.n_layers
    kv = {}
    for layer in (0, L - 1):
        for kind in ("k", "v"):
            kv[f"{kind}_cache_layer{layer}"] = m.kv_read(layer, kind, rows)[pick].astype(np.float32)
    np.savez_compressed(os.path.join(HERE, f"{name}_full.npz"), config=cfg, seed=seed, prompt=np.array(prompt, dtype=np.int32),
                        tokens=np.array(toks, dtype=np.int32), margins=np.array(margins, dtype=np.float32),
                        prompt_logits=prompt_logits.astype(np.float32), last_logits=logits.astype(np.float32),
                        cache_rows=np.array(pick, dtype=np.int32), **kv)
    print(name, "tokens", toks, "min margin", float(min(margins)), "max |logit|", float(np.max(np.abs(logits))),
          f"({time.time() - t0:.0f} s)", flush=True)


# batched decode on the whole Llama-3-8B-shape model: sequences of different lengths decoded side by side, one row each per step.
# The oracle runs them one after the other (they do not interact).  name: (config, seed, first prompt length, sequences, steps)
BATCH_CASES = {
    "llama3_8b_q8_batch4": ("llama3_8b_q8", FULL_SEED, 256, 4, 16),
}


def batch_case(pkg, name):
    cfg, seed, n_prompt, n_seq, n_new = BATCH_CASES[name]
    d = pkg.CONFIGS[cfg].copy(max_seq=n_prompt + n_seq + n_new + 8)
    t0 = time.time()
    m = OracleModel(d)
    m.synth(seed)
    base = m.synth_tokens(seed, n_prompt + n_seq)
    prompts, toks, margins, last = [], [], [], []
    for sq in range(n_seq):
        prompt = base[sq:sq + n_prompt + sq // 2]             # different lengths: 256, 256, 257, 257 tokens, shifted starts
        t, logits, mg = m.generate(prompt, n_new + 1, return_last_logits=True, return_margins=True)
        prompts.append(np.array(prompt, dtype=np.int32)); toks.append(t); margins.append(mg); last.append(logits.astype(np.float32))
        print(f"{name}: sequence {sq} done after {time.time() - t0:.0f} s, min margin {min(mg):.3e}", flush=True)
    np.savez_compressed(os.path.join(HERE, f"{name}_full.npz"), config=cfg, seed=seed, n_seq=n_seq,
                        prompt_lens=np.array([len(p) for p in prompts], dtype=np.int32), prompts=np.concatenate(prompts),
                        tokens=np.array(toks, dtype=np.int32), margins=np.array(margins, dtype=np.float32), last_logits=np.stack(last))
    print(name, "tokens", toks, f"({time.time() - t0:.0f} s)", flush=True)


def main():
    pkg = load_package()
    wanted = sys.argv[1:]
    if wanted:
        for name in wanted:
            if name in BATCH_CASES:
                batch_case(pkg, name)
            else:
                full_case(pkg, name)
        return
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
