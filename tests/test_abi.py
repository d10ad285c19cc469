"""CPU tests of the boundary: the library builds for sm_100a, exports every symbol the header declares,
refuses to run without a GPU (no CPU fallback), and the host-side helpers agree with the stated byte counts."""
import ctypes as C
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "lum_b200.h")


@pytest.fixture(scope="module")
def lib(pkg):
    if not os.path.exists(pkg.library_path()):
        if shutil.which("nvcc") is None:
            pytest.skip("library not built and nvcc unavailable")
        subprocess.run(["make", "-j", "4", "-C", os.path.join(ROOT, "oneiron-luminal_b200", "csrc")], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return pkg.load_library()


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lum_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_expected_surface():
    syms = declared_symbols()
    for must in ["lum_create", "lum_destroy", "lum_model_init", "lum_set_dim", "lum_set_tokens", "lum_execute",
                 "lum_get_logits", "lum_profile", "lum_kv_reset", "lum_decode_greedy", "lum_op_gemv_q8_0"]:
        assert must in syms
    # the boundary a `Runtime` implementation over this library binds (src/op.rs:10-30 and the inherent methods of
    # crates/luminal_cuda/src/runtime.rs:133-236): graph in, inputs by node id (host data or a caller's device pointer), dynamic
    # dimensions, the search's dummy inputs / clear / profile of a graph, outputs in f32 or their own type, the sampled token,
    # cache handling, errors and counters
    for must in ["lum_load_llir", "lum_llir_describe", "lum_set_input", "lum_set_input_device_ptr", "lum_alloc_dummy_input",
                 "lum_clear_intermediates", "lum_profile_llir", "lum_get_output", "lum_get_output_raw", "lum_get_token", "lum_kv_read",
                 "lum_kv_save", "lum_kv_load", "lum_kv_copy", "lum_kv_release", "lum_kv_pool", "lum_last_error", "lum_get_stats",
                 "lum_load_safetensors", "lum_save_safetensors", "lum_model_set_weight", "lum_model_set_weight_shard",
                 "lum_seq_select", "lum_batch_begin", "lum_batch_begin_slots", "lum_batch_decode", "lum_batch_get_decoded",
                 "lum_set_sampling", "lum_op_sample_topk", "lum_op_sample_q8_0_static", "lum_op_status",
                 "lum_tp_unique_id", "lum_tp_init", "lum_tp_peer_export", "lum_tp_peer_import", "lum_synchronize"]:
        assert must in syms, must


def test_library_exports_every_declared_symbol(lib):
    raw = C.CDLL(lib._name)
    missing = [s for s in declared_symbols() if not hasattr(raw, s)]
    assert not missing, f"declared in lum_b200.h but not exported: {missing}"


def test_no_cpu_fallback(lib, pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.LumError) as ei:
        pkg.B200Runtime.initialize(device=0)
    assert "no CPU fallback" in str(ei.value) or "CUDA" in str(ei.value)


def test_missing_library_fails_loudly(pkg, monkeypatch, tmp_path):
    from oneiron_luminal_b200 import runtime
    monkeypatch.setattr(runtime, "_lib", None)
    monkeypatch.setattr(runtime, "_HERE", str(tmp_path))
    with pytest.raises(pkg.LumError, match="not built"):
        runtime.load_library()


def test_decode_byte_model_matches_stated_figures(pkg):
    d = pkg.CONFIGS["llama3_8b_q8"]
    # 7,504,658,432 weights x 34/32 + gains 532,480 + one embedding row 8,192 + 131,072 per KV row
    assert pkg.decode_bytes_per_token(d, 512) == 8_041_480_192
    assert pkg.decode_bytes_per_token(d, 640) == 8_058_257_408
    assert pkg.decode_bytes_per_token(d, 0) == 7_974_240_256 + 131_072


def test_llir_blob_layout(pkg):
    import struct
    from oneiron_luminal_b200 import llir
    b = llir.LLIRBuilder()
    a = b.input(7, "tok", 3)
    b.output(a, 9)
    blob = b.blob()
    magic, ver, n = struct.unpack_from("<III", blob)
    assert (magic, ver, n) == (0x52494C4C, 1, 2)
    assert blob[12:12 + 4 + 5] == struct.pack("<I", 5) + b"Input"
    # z - 3: right operand first, left operand last, then the operator
    e = llir.Expr.of("z") - 3
    assert e.terms == [(llir.T_NUM, 3), (llir.T_VAR, ord("z")), (llir.T_SUB, 0)]
