"""Host-side checks of bench.py that need no GPU: the CPU arm with many steps, the seeded prompt."""
import json

import numpy as np


def test_reference_arm_with_many_steps(pkg, monkeypatch, capsys):
    """`bench.py --impl reference --steps 20 --warmup 5` on a small stand-in workload:
    25 single-token passes must fit the oracle's cache and print one well-formed JSON line."""
    import bench
    monkeypatch.setattr(bench, "WORKLOAD", "small_q8")
    monkeypatch.setattr(bench, "PROMPT_LEN", 16)
    monkeypatch.setattr(bench, "TOKENS_PER_STEP", 4)

    class Args:
        steps, warmup, gpus = 20, 5, 1

    bench.run_reference_arm(Args, pkg)
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["value"] > 0 and line["scaling"] == "strong"
    assert line["config"] == bench.bench_config(1, 5, True) | {"note": line["config"]["note"]}
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["value"] == line["value"]
    assert abs(line["ms_per_step"] * line["value"] - 1000.0) < 1e-6


def test_prompt_generator_matches_the_oracle(pkg):
    import bench
    from oracle import OracleModel
    d = pkg.CONFIGS["small_q8"]
    m = OracleModel(d)
    assert bench._prompt_tokens(d.vocab, 64) == m.synth_tokens(bench.SEED, 64)


def test_full_size_fixtures_are_for_the_bench_seed_and_prompt(pkg):
    """The committed whole-model fixtures must be the benchmark's own seed and prompt, or bench.py's parity object is void."""
    import os
    import bench
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    for name, n_prompt in (("llama3_8b_q8", 512), ("qwen3_4b_q8", 1024)):
        path = os.path.join(here, f"{name}_full.npz")
        if not os.path.exists(path):
            continue
        fx = np.load(path)
        d = pkg.CONFIGS[name]
        assert int(fx["seed"]) == bench.SEED
        assert list(fx["prompt"]) == bench._prompt_tokens(d.vocab, n_prompt)
        assert fx["tokens"].size == 32 and fx["prompt_logits"].size == d.vocab and fx["margins"].size == 32
