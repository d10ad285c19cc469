"""The C++ host (oneiron-luminal_b200/host/b200_runtime.hpp, header-only over the C ABI) compiled with g++ and driven by
tests/host_cpp/drive.cpp.  Without a GPU: it compiles, links against the library and the host-only entries work.  On a GPU: it
decodes the same tokens as the Python host from the same description bytes, and runs a graph of primitive ops."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def drive(pkg, tmp_path_factory):
    out = str(tmp_path_factory.mktemp("host_cpp") / "drive")
    libdir = os.path.dirname(pkg.library_path())
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "host_cpp", "drive.cpp"),
           "-o", out, "-L", libdir, "-llum_b200", f"-Wl,-rpath,{libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return out


def test_cpp_host_compiles_links_and_runs_host_only_entries(pkg, drive, tmp_path):
    from oneiron_luminal_b200 import llir
    desc = pkg.CONFIGS["small_q8"]
    blob, ids = llir.build_llama_llir(desc)
    g = tmp_path / "g.llir"
    g.write_bytes(blob)
    st = tmp_path / "t.safetensors"
    r = subprocess.run([drive, "abi", str(g), str(st)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.splitlines()
    assert lines[0] == "config use_graph=1 use_pdl=1"
    assert f"describe rc=0 layers={desc.n_layers} hidden={desc.hidden} vocab={desc.vocab}" in lines[1]
    assert lines[2] == "tensor w dtype=0 shape=2x3 bytes=24 last=6 meta=drive.cpp"
    got, _ = pkg.safetensors_read(str(st))
    assert np.array_equal(got["w"][1], np.arange(1, 7, dtype=np.float32).reshape(2, 3))


@pytest.mark.gpu
def test_cpp_host_decodes_what_the_python_host_decodes(pkg, drive, tmp_path):
    desc = pkg.CONFIGS["small_q8"]
    prompt = [11, 22, 33, 44, 55, 66]
    rt = pkg.B200Runtime.initialize(device=0)
    try:
        rt.load_model(desc); rt.synth(5)
        want = rt.generate(prompt, 12)
    finally:
        rt.close()
    d = tmp_path / "desc.bin"
    d.write_bytes(bytes(desc))
    r = subprocess.run([drive, "decode", str(d), "5", "12"] + [str(t) for t in prompt], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.splitlines()
    assert lines[0] == "tokens " + " ".join(str(t) for t in want)
    assert lines[1].startswith(f"logits {desc.vocab} launches_per_step ")
    assert lines[2] == "caught -1"


@pytest.mark.gpu
def test_cpp_host_runs_a_primitive_graph(pkg, drive, tmp_path):
    from oneiron_luminal_b200 import llir as L
    n = 9
    b = L.LLIRBuilder()
    a = b.input(0, "a", 0)
    b.output(b.unary("Sqrt", [n], b.binary("Mul", [n], a, [1], a, [1]), [1]), 2)
    g = tmp_path / "p.llir"
    g.write_bytes(b.blob())
    r = subprocess.run([drive, "graph", str(g), str(n)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.split() == ["out"] + [str(i) for i in range(n)]


def test_cpp_serving_loop_on_a_stand_in_runtime(tmp_path):
    """oneiron-luminal_b200/host/serving.hpp (the continuous-batching loop in C++) against a stand-in runtime: results equal
    each request alone, end-of-sequence ids, parked prefixes, page-aware admission, refusals."""
    out = str(tmp_path / "serving_test")
    r = subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", os.path.join(ROOT, "tests", "host_cpp", "serving_test.cpp"), "-o", out],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([out], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip() == "ok 5", r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_serving_loop_equals_requests_alone(pkg, drive, tmp_path):
    """The C++ loop over the real runtime with a paged cache: five requests through three slots get the tokens they get alone."""
    desc = pkg.CONFIGS["llama3_8b_q8_2layer"].copy(max_batch=3, max_seq=256, max_new_tokens=64, kv_page_rows=64, kv_pool_pages=7)
    spec = [(5, 9), (70, 30), (40, 13), (9, 1), (100, 20)]
    solo = pkg.B200Runtime.initialize(device=0)
    try:
        solo.load_model(desc.copy(max_batch=1, kv_page_rows=0, kv_pool_pages=0)); solo.synth(77)
        alone = [solo.generate([(11 * k + 5 * i + 1) % desc.vocab for k in range(n)], m) for i, (n, m) in enumerate(spec)]
    finally:
        solo.close()
    d = tmp_path / "desc.bin"
    d.write_bytes(bytes(desc))
    r = subprocess.run([drive, "serve", str(d), "77"] + [f"{n}:{m}" for n, m in spec], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.splitlines()
    for i, want in enumerate(alone):
        assert lines[i] == f"request {i}: " + " ".join(str(t) for t in want), i
    assert lines[len(spec)].startswith("pool 7 7 64 rows_per_step ")
