"""ctypes host for ``liblum_b200.so`` — mirrors the reference's runtime surface.

Reference interface -> method here
  ``Runtime::initialize(arg)``          src/op.rs:15                 -> ``B200Runtime.initialize(device=…)``
  ``Runtime::execute(&dyn_map)``        src/op.rs:17                 -> ``execute({'s': n, 'p': prev})``
  ``Runtime::profile(..)``              src/op.rs:18-23              -> ``profile(trials)``
  ``CudaRuntime::set_data(id, data)``   luminal_cuda runtime.rs:160  -> ``set_data(token_ids)`` / ``set_weight(..)``
  ``CudaRuntime::get_f32(id)``          luminal_cuda runtime.rs:168  -> ``get_f32()`` (logits of the last row)
  ``KVCache::reset``                    examples/llama/src/model.rs:217 -> ``kv_reset()``
  ``sample``                            examples/llama/src/main.rs:137  -> ``get_token()`` (device-side greedy)
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Iterable, Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_NAME = "liblum_b200.so"


class LumError(RuntimeError):
    """A C-ABI call returned a non-zero status; ``code`` is the LUM_E_* value."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"[lum {code}] {msg}")
        self.code = code


DTYPE = {"f32": 0, "f16": 1, "bf16": 2, "int": 3, "bool": 4, "nvfp4": 5, "mxfp4": 6, "q8_0": 7}
SLOT = {
    "embed": 0, "attn_norm": 1, "q": 2, "k": 3, "v": 4, "o": 5, "mlp_norm": 6,
    "gate": 7, "up": 8, "down": 9, "final_norm": 10, "lm_head": 11, "q_norm": 12, "k_norm": 13,
    "q_bias": 14, "k_bias": 15, "v_bias": 16, "o_bias": 17, "sinks": 18, "router": 19, "router_bias": 20,
    "exp_gate_up": 21, "exp_gate_up_bias": 22, "exp_down": 23, "exp_down_bias": 24,
}


class Config(C.Structure):
    _fields_ = [("device", C.c_int32), ("use_graph", C.c_int32), ("use_pdl", C.c_int32), ("attn_splits", C.c_int32),
                ("use_mega", C.c_int32), ("prefill_min_rows", C.c_int32), ("wait_budget_ms", C.c_int32)]


class ModelDesc(C.Structure):
    """Mirror of ``lum_model_desc`` (include/lum_b200.h)."""

    _fields_ = [
        ("n_layers", C.c_int32), ("hidden", C.c_int32), ("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32), ("max_seq", C.c_int32),
        ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("rope_style", C.c_int32),
        ("weight_dtype", C.c_uint32), ("embed_dtype", C.c_uint32), ("kv_dtype", C.c_uint32),
        ("qk_norm", C.c_int32), ("tied_head", C.c_int32), ("max_new_tokens", C.c_int32),
        ("tp_size", C.c_int32), ("tp_rank", C.c_int32), ("max_batch", C.c_int32),
        ("sliding_window", C.c_int32), ("window_even_layers", C.c_int32), ("attn_sinks", C.c_int32), ("proj_bias", C.c_int32),
        ("yarn_factor", C.c_float), ("yarn_beta_fast", C.c_float), ("yarn_beta_slow", C.c_float), ("yarn_orig_max_pos", C.c_float),
        ("n_experts", C.c_int32), ("top_k", C.c_int32), ("swiglu_limit", C.c_float), ("ep_size", C.c_int32), ("ep_rank", C.c_int32),
        ("kv_page_rows", C.c_int32), ("kv_pool_pages", C.c_int32),
    ]

    def copy(self, **kw) -> "ModelDesc":
        d = ModelDesc()
        C.memmove(C.byref(d), C.byref(self), C.sizeof(ModelDesc))
        for k, v in kw.items():
            setattr(d, k, v)
        return d


class Stats(C.Structure):
    """Mirror of ``lum_stats`` (include/lum_b200.h)."""

    _fields_ = [("tokens_executed", C.c_uint64), ("kernel_launches", C.c_uint64), ("weight_bytes_per_token", C.c_uint64),
                ("kv_bytes_per_position", C.c_uint64), ("launches_per_step", C.c_int32), ("reserved", C.c_int32),
                ("last_profile_usec", C.c_double)]


class Sampling(C.Structure):
    """Mirror of ``lum_sampling`` (include/lum_b200.h): temperature / top-p / top-k / seed of the on-device sampler."""

    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int32), ("reserved", C.c_int32), ("seed", C.c_uint64)]


def _desc(**kw) -> ModelDesc:
    d = ModelDesc()
    base = dict(max_seq=4096, rms_eps=1e-5, rope_style=0, qk_norm=0, tied_head=0, max_new_tokens=4096, tp_size=1, tp_rank=0, max_batch=1)
    base.update(kw)
    for k, v in base.items():
        setattr(d, k, v)
    return d


# The workloads this runtime is measured and tested on (shapes only; weights are synthetic).
CONFIGS: Dict[str, ModelDesc] = {
    # tiny all-f32 decoder, CPU-runnable by the reference's interpreter
    "tiny_f32": _desc(n_layers=2, hidden=256, n_q_heads=4, n_kv_heads=2, head_dim=64, ffn=688, vocab=1024, max_seq=64,
                      rope_theta=10000.0, weight_dtype=DTYPE["f32"], embed_dtype=DTYPE["f32"], kv_dtype=DTYPE["f32"]),
    # Llama-3-8B shape, Q8_0 linears, bf16 embedding / gains / KV cache
    "llama3_8b_q8": _desc(n_layers=32, hidden=4096, n_q_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, vocab=128256,
                          max_seq=4096, rope_theta=500000.0, weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"],
                          kv_dtype=DTYPE["bf16"]),
    # a 2-layer cut of the same shape with a small vocabulary: same kernels and tile shapes, seconds on a CPU
    "llama3_8b_q8_2layer": _desc(n_layers=2, hidden=4096, n_q_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, vocab=4096,
                                 max_seq=256, rope_theta=500000.0, weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"],
                                 kv_dtype=DTYPE["bf16"]),
    # Qwen3-4B shape: per-head q/k RMSNorm, split-half RoPE, theta 1e6, eps 1e-6, head tied to the bf16 embedding
    "qwen3_4b_q8": _desc(n_layers=36, hidden=2560, n_q_heads=32, n_kv_heads=8, head_dim=128, ffn=9728, vocab=151936,
                         max_seq=4096, rms_eps=1e-6, rope_theta=1000000.0, rope_style=1, qk_norm=1, tied_head=1,
                         weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"], kv_dtype=DTYPE["bf16"]),
    # Qwen3-4B layer shape (per-head q/k RMSNorm, split-half RoPE, theta 1e6, eps 1e-6, head tied to the embedding) cut to
    # 2 layers and a small vocabulary: hidden 2560 = 5 tiles, ffn 9728 = 19 tiles per row group
    "qwen3_4b_q8_2layer": _desc(n_layers=2, hidden=2560, n_q_heads=32, n_kv_heads=8, head_dim=128, ffn=9728, vocab=4096,
                                max_seq=256, rms_eps=1e-6, rope_theta=1000000.0, rope_style=1, qk_norm=1, tied_head=1,
                                weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"], kv_dtype=DTYPE["bf16"]),
    # like small_q8, but with an FFN width whose half (1792 = 3.5 tiles) does not cut into tiles: sharded over two ranks, the
    # down and o projections take the plain-load kernel — the shapes an 8-way split of the Llama-3-8B model produces
    "small_q8_odd": _desc(n_layers=2, hidden=512, n_q_heads=8, n_kv_heads=2, head_dim=64, ffn=3584, vocab=2048, max_seq=128,
                          rope_theta=500000.0, weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"], kv_dtype=DTYPE["bf16"]),
    # a quarter of the Llama-3-8B layer (8/2 heads, ffn 3584, vocabulary 32064) at full hidden size: split over 2 ranks, every
    # rank holds exactly the shard shapes of the full model split over 8 (one KV head, o K = 512, down K = 1792, 16032 vocabulary rows)
    "llama3_8b_q8_quarter": _desc(n_layers=2, hidden=4096, n_q_heads=8, n_kv_heads=2, head_dim=128, ffn=3584, vocab=32064,
                                  max_seq=256, rope_theta=500000.0, weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"],
                                  kv_dtype=DTYPE["bf16"]),
    # gpt-oss-20B shape (examples/gpt_oss scaled to 24 layers / 32 experts): alternating 128-token sliding-window and full layers,
    # per-head sinks, projection biases, YaRN RoPE, top-4 of 32 experts of width 2880
    "gpt_oss_20b_q8": _desc(n_layers=24, hidden=2880, n_q_heads=64, n_kv_heads=8, head_dim=64, ffn=2880, vocab=201088, max_seq=4096,
                            rope_theta=150000.0, rope_style=2, weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"], kv_dtype=DTYPE["bf16"],
                            sliding_window=128, window_even_layers=1, attn_sinks=1, proj_bias=1, yarn_factor=32.0, yarn_beta_fast=32.0,
                            yarn_beta_slow=1.0, yarn_orig_max_pos=4096.0, n_experts=32, top_k=4, swiglu_limit=7.0),
    # the same layer kind, small: window 8 so that a short run leaves it, 16/2 heads of 64 (8 query heads per KV head), 8 experts
    "small_oss": _desc(n_layers=4, hidden=512, n_q_heads=16, n_kv_heads=2, head_dim=64, ffn=512, vocab=2048, max_seq=128,
                       rope_theta=150000.0, rope_style=2, weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"], kv_dtype=DTYPE["bf16"],
                       sliding_window=8, window_even_layers=1, attn_sinks=1, proj_bias=1, yarn_factor=32.0, yarn_beta_fast=32.0,
                       yarn_beta_slow=1.0, yarn_orig_max_pos=4096.0, n_experts=8, top_k=4, swiglu_limit=7.0),
    # the gpt-oss-20B layer's own awkward sizes, small: hidden 576 and expert width 352 are whole 32-blocks but not whole tiles, and the
    # per-expert activation block of the down kernel (3 * 352 + 44 = 1100 bytes) is not a multiple of 16 (2880: 9000 bytes, the same class)
    "small_oss_352": _desc(n_layers=2, hidden=576, n_q_heads=16, n_kv_heads=2, head_dim=64, ffn=352, vocab=2048, max_seq=128,
                           rope_theta=150000.0, rope_style=2, weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"], kv_dtype=DTYPE["bf16"],
                           sliding_window=8, window_even_layers=1, attn_sinks=1, proj_bias=1, yarn_factor=32.0, yarn_beta_fast=32.0,
                           yarn_beta_slow=1.0, yarn_orig_max_pos=4096.0, n_experts=8, top_k=4, swiglu_limit=7.0),
    # the attention features alone on a dense FFN (window, sinks, biases, YaRN), hidden not a multiple of the tile width
    "small_oss_dense": _desc(n_layers=3, hidden=576, n_q_heads=16, n_kv_heads=2, head_dim=64, ffn=1152, vocab=2048, max_seq=128,
                             rope_theta=150000.0, rope_style=2, weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"], kv_dtype=DTYPE["bf16"],
                             sliding_window=8, window_even_layers=1, attn_sinks=1, proj_bias=1, yarn_factor=32.0, yarn_beta_fast=32.0,
                             yarn_beta_slow=1.0, yarn_orig_max_pos=4096.0),
    # small Q8_0 model for fast parity runs
    "small_q8": _desc(n_layers=3, hidden=512, n_q_heads=8, n_kv_heads=2, head_dim=64, ffn=1536, vocab=2048, max_seq=128,
                      rope_theta=500000.0, weight_dtype=DTYPE["q8_0"], embed_dtype=DTYPE["bf16"], kv_dtype=DTYPE["bf16"]),
}


def decode_bytes_per_token(d: ModelDesc, p: float) -> float:
    """Algorithmic HBM bytes one decode step must move with ``p`` tokens already cached:
    every linear weight once (Q8_0 = 34/32 B per weight), norm gains, one embedding row, the KV rows read and
    the one row written.  Activations are excluded."""
    wb = 34.0 / 32.0 if d.weight_dtype == DTYPE["q8_0"] else 4.0
    eb = 2.0 if d.embed_dtype == DTYPE["bf16"] else 4.0
    kb = 2.0 if d.kv_dtype == DTYPE["bf16"] else 4.0
    qd, kvd = d.n_q_heads * d.head_dim, d.n_kv_heads * d.head_dim
    per_layer = (qd * d.hidden + 2 * kvd * d.hidden + d.hidden * qd + 3 * d.ffn * d.hidden)
    head = d.vocab * d.hidden
    weights = d.n_layers * per_layer * wb + (head * eb if d.tied_head else head * wb)
    gains = (2 * d.n_layers + 1) * d.hidden * eb
    kv_row = d.n_layers * 2 * kvd * kb
    return weights + gains + d.hidden * eb + kv_row * (p + 1)


def library_path() -> str:
    return os.path.join(_HERE, _LIB_NAME)


_lib = None


def load_library() -> C.CDLL:
    """Load the built C-ABI library; raises (never falls back) when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise LumError(-3, f"{path} is not built; run `make -C {os.path.join(_HERE, 'csrc')}` (needs nvcc) — there is no CPU fallback")
    lib = C.CDLL(path)
    i32, u32, u64, sz, vp = C.c_int32, C.c_uint32, C.c_uint64, C.c_size_t, C.c_void_p
    P = C.POINTER
    sig = {
        "lum_config_default": (None, [P(Config)]),
        "lum_create": (i32, [P(Config), P(vp)]),
        "lum_destroy": (None, [vp]),
        "lum_last_error": (C.c_char_p, [vp]),
        "lum_device_info": (i32, [vp, P(i32), P(u64), P(i32)]),
        "lum_model_init": (i32, [vp, P(ModelDesc)]),
        "lum_model_set_weight": (i32, [vp, i32, i32, vp, sz, u32]),
        "lum_model_set_weight_shard": (i32, [vp, i32, i32, vp, sz, u32]),
        "lum_load_safetensors": (i32, [vp, C.c_char_p, P(i32), P(i32)]),
        "lum_save_safetensors": (i32, [vp, C.c_char_p]),
        "lum_op_q8_0_quantize": (i32, [vp, u32, sz, vp, vp, vp]),
        "lum_st_last_error": (C.c_char_p, []),
        "lum_st_open": (i32, [C.c_char_p, P(vp)]),
        "lum_st_close": (None, [vp]),
        "lum_st_count": (i32, [vp]),
        "lum_st_tensor": (i32, [vp, i32, P(C.c_char_p), P(u32), P(i32), P(C.c_int64), P(vp), P(sz)]),
        "lum_st_metadata": (C.c_char_p, [vp, C.c_char_p]),
        "lum_st_write": (i32, [C.c_char_p, i32, P(C.c_char_p), P(u32), P(i32), P(C.c_int64), P(vp), i32, P(C.c_char_p), P(C.c_char_p)]),
        "lum_model_synth": (i32, [vp, u64]),
        "lum_model_get_weight_f32": (i32, [vp, i32, i32, sz, sz, P(C.c_float)]),
        "lum_model_weight_bytes": (i32, [vp, P(u64)]),
        "lum_llir_describe": (i32, [vp, sz, P(ModelDesc), P(C.c_int64), P(C.c_int64), P(C.c_int64), C.c_char_p, sz]),
        "lum_load_llir": (i32, [vp, vp, sz, i32, u32, i32]),
        "lum_set_input": (i32, [vp, C.c_int64, vp, sz, u32]),
        "lum_set_input_device_ptr": (i32, [vp, C.c_int64, vp, sz, u32]),
        "lum_alloc_dummy_input": (i32, [vp, C.c_int64, sz]),
        "lum_clear_intermediates": (i32, [vp]),
        "lum_profile_llir": (i32, [vp, vp, sz, u64, u64, i32, P(C.c_double), C.c_char_p, sz]),
        "lum_llir_describe_chunk": (i32, [vp, sz, P(ModelDesc), P(C.c_int64), P(C.c_int64), C.c_char_p, sz]),
        "lum_kv_save": (i32, [vp, i32, i32, i32, vp, sz]),
        "lum_kv_load": (i32, [vp, i32, i32, i32, vp, sz]),
        "lum_kv_copy": (i32, [vp, i32, i32, i32]),
        "lum_kv_release": (i32, [vp, i32]),
        "lum_kv_pool": (i32, [vp, P(i32), P(i32), P(i32)]),
        "lum_set_sampling": (i32, [vp, P(Sampling)]),
        "lum_op_sample_topk": (i32, [vp, i32, i32, P(Sampling), i32, vp, vp, vp]),
        "lum_get_stats": (i32, [vp, P(Stats)]),
        "lum_debug_wait_timeout": (i32, [vp]),
        "lum_op_status": (i32, [vp]),
        "lum_get_output": (i32, [vp, C.c_int64, P(C.c_float), sz]),
        "lum_get_output_raw": (i32, [vp, C.c_int64, vp, sz, P(u32), P(sz)]),
        "lum_kv_reset": (i32, [vp]),
        "lum_kv_read": (i32, [vp, i32, i32, i32, P(C.c_float)]),
        "lum_set_dim": (i32, [vp, C.c_char, u64]),
        "lum_set_tokens": (i32, [vp, P(i32), sz]),
        "lum_execute": (i32, [vp]),
        "lum_get_logits": (i32, [vp, P(C.c_float), sz]),
        "lum_get_token": (i32, [vp, P(i32)]),
        "lum_decode_greedy": (i32, [vp, i32]),
        "lum_get_decoded": (i32, [vp, P(i32), sz]),
        "lum_decode_reset": (i32, [vp]),
        "lum_synchronize": (i32, [vp]),
        "lum_seq_select": (i32, [vp, i32]),
        "lum_batch_begin": (i32, [vp, i32, P(i32), P(i32)]),
        "lum_batch_begin_slots": (i32, [vp, i32, P(i32), P(i32), P(i32)]),
        "lum_batch_decode": (i32, [vp, i32]),
        "lum_batch_get_decoded": (i32, [vp, P(i32), sz]),
        "lum_batch_get_logits": (i32, [vp, i32, P(C.c_float), sz]),
        "lum_profile": (i32, [vp, i32, P(C.c_double), C.c_char_p, sz]),
        "lum_launches_per_step": (i32, [vp, P(i32)]),
        "lum_stream": (vp, [vp]),
        "lum_tp_unique_id": (i32, [vp]),
        "lum_tp_init": (i32, [vp, vp, i32, i32]),
        "lum_tp_peer_export": (i32, [vp, vp]),
        "lum_tp_peer_import": (i32, [vp, vp, i32]),
        "lum_op_gemv_q8_0": (i32, [vp, vp, i32, i32, vp, vp, i32, vp]),
        "lum_q8_0_packed_bytes": (sz, [i32, i32]),
        "lum_op_q8_0_pack": (i32, [vp, vp, i32, i32, vp, vp]),
        "lum_op_gemv_q8_0_packed": (i32, [vp, i32, i32, vp, vp, i32, vp]),
        "lum_op_synth_q8_0_packed": (i32, [u64, u64, i32, i32, vp, vp]),
        "lum_op_gemm_q8_0_workspace": (sz, [i32, i32, i32]),
        "lum_op_gemm_q8_0_packed": (i32, [vp, i32, i32, vp, i32, vp, vp, sz, vp]),
        "lum_op_sample_q8_0": (i32, [vp, i32, i32, vp, vp, vp, vp]),
        "lum_op_sample_q8_0_static": (i32, [vp, i32, i32, vp, vp, vp, vp]),
        "lum_op_gemv_f32": (i32, [vp, i32, i32, vp, vp, vp]),
        "lum_op_q8_0_unpack": (i32, [vp, sz, vp, vp, vp]),
        "lum_op_q8_0_dequant": (i32, [vp, vp, sz, vp, vp]),
        "lum_op_synth_q8_0": (i32, [u64, u64, sz, vp, vp, vp]),
        "lum_op_synth_normal": (i32, [u64, u64, u32, sz, i32, vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)   # AttributeError here = header and library disagree: fail loudly
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


EXPORTED_SYMBOLS = None  # filled lazily by tests from include/lum_b200.h


_ST_NP = {0: "float32", 1: "float16", 2: "uint16", 3: "int32", 4: "bool", 100: "uint8"}      # bf16 values travel as their bit patterns


def safetensors_read(path: str):
    """Host-only: ``(tensors, metadata)`` of a safetensors file through the library's own reader.  ``tensors`` maps a name to
    ``(dtype_name, numpy array)``; bf16 tensors come back as uint16 bit patterns (dtype_name "bf16"); dtypes the library does
    not read come back as ``("other", raw uint8 bytes)``."""
    import numpy as np
    lib = load_library()
    h = C.c_void_p()
    if lib.lum_st_open(path.encode(), C.byref(h)):
        raise LumError(-1, lib.lum_st_last_error().decode())
    try:
        out = {}
        for i in range(lib.lum_st_count(h)):
            name, dt, nd, n = C.c_char_p(), C.c_uint32(), C.c_int32(), C.c_size_t()
            shape = (C.c_int64 * 8)()
            data = C.c_void_p()
            if lib.lum_st_tensor(h, i, C.byref(name), C.byref(dt), C.byref(nd), shape, C.byref(data), C.byref(n)):
                raise LumError(-1, lib.lum_st_last_error().decode())
            raw = np.frombuffer(C.string_at(data, n.value), dtype=np.uint8) if n.value else np.zeros(0, np.uint8)
            dims = tuple(int(shape[k]) for k in range(nd.value))
            if dt.value in _ST_NP:
                arr = raw.view(_ST_NP[dt.value]).reshape(dims)
                out[name.value.decode()] = ({0: "f32", 1: "f16", 2: "bf16", 3: "i32", 4: "bool", 100: "u8"}[dt.value], arr)
            else:
                out[name.value.decode()] = ("other", raw)
        meta = {}
        for k in ("lum.shard", "lum.tp_size", "lum.tp_rank", "lum.ep_size", "lum.ep_rank", "lum.q8_0", "format"):
            v = lib.lum_st_metadata(h, k.encode())
            if v is not None:
                meta[k] = v.decode()
        return out, meta
    finally:
        lib.lum_st_close(h)


def safetensors_write(path: str, tensors, metadata=None) -> None:
    """Host-only: write ``{name: (dtype_name, numpy array)}`` (dtype names as safetensors_read returns them) with the library's
    own writer; tensors are stored in the order given."""
    import numpy as np
    lib = load_library()
    code = {"f32": 0, "f16": 1, "bf16": 2, "i32": 3, "bool": 4, "u8": 100}
    names = list(tensors)
    n = len(names)
    arrs = [np.require(tensors[k][1], requirements="C") for k in names]        # (ascontiguousarray would turn a scalar into [1])
    c_names = (C.c_char_p * n)(*[k.encode() for k in names])
    c_dt = (C.c_uint32 * n)(*[code[tensors[k][0]] for k in names])
    c_nd = (C.c_int32 * n)(*[a.ndim for a in arrs])
    c_sh = (C.c_int64 * (8 * n))()
    for i, a in enumerate(arrs):
        for k, d in enumerate(a.shape):
            c_sh[8 * i + k] = d
    c_data = (C.c_void_p * n)(*[a.ctypes.data for a in arrs])
    md = dict(metadata or {})
    mk = (C.c_char_p * max(1, len(md)))(*[k.encode() for k in md])
    mv = (C.c_char_p * max(1, len(md)))(*[str(v).encode() for v in md.values()])
    if lib.lum_st_write(path.encode(), n, c_names, c_dt, c_nd, c_sh, c_data, len(md), mk, mv):
        raise LumError(-1, lib.lum_st_last_error().decode())


def describe_llir(blob: bytes):
    """Host-only: ``(ModelDesc, token_input, pos_input, logits_output)`` a serialised graph implies; raises
    ``LumError`` naming the node where the graph stops looking like a Llama-style decoder."""
    lib = load_library()
    d = ModelDesc()
    tok, pos, out = C.c_int64(-1), C.c_int64(-1), C.c_int64(-1)
    err = C.create_string_buffer(256)
    buf = C.create_string_buffer(blob, len(blob))
    rc = lib.lum_llir_describe(buf, len(blob), C.byref(d), C.byref(tok), C.byref(pos), C.byref(out), err, 256)
    if rc != 0:
        raise LumError(rc, err.value.decode())
    return d, tok.value, pos.value, out.value


def describe_llir_chunk(blob: bytes):
    """Host-only: ``(ModelDesc, hidden_input, hidden_output)`` of a chunk of whole layers (what the reference's search
    profiles between two GraphBreaks); raises ``LumError`` for anything else."""
    lib = load_library()
    d = ModelDesc()
    hin, hout = C.c_int64(-1), C.c_int64(-1)
    err = C.create_string_buffer(256)
    buf = C.create_string_buffer(blob, len(blob))
    rc = lib.lum_llir_describe_chunk(buf, len(blob), C.byref(d), C.byref(hin), C.byref(hout), err, 256)
    if rc != 0:
        raise LumError(rc, err.value.decode())
    return d, hin.value, hout.value


def mbu(stats: "Stats", usec_per_token: float, context: int, peak_gb_s: float) -> float:
    """Memory-bandwidth utilisation of a decode step, the way the reference's bench crate states it
    (crates/luminal_bench/src/metrics.rs:13-60): bytes the step must move / time / peak bandwidth."""
    bytes_tok = stats.weight_bytes_per_token + stats.kv_bytes_per_position * (context + 1)
    return bytes_tok / (usec_per_token * 1e-6) / (peak_gb_s * 1e9)


class B200Runtime:
    """One runtime = one B200 = one stream (as `CudaRuntime`, crates/luminal_cuda/src/runtime.rs:87-131)."""

    def __init__(self, handle: int, lib: C.CDLL):
        self._h = C.c_void_p(handle)
        self._lib = lib
        self.desc: Optional[ModelDesc] = None

    # ---- lifecycle -------------------------------------------------------------------------------
    @classmethod
    def initialize(cls, device: int = 0, use_graph: Optional[bool] = None, use_pdl: Optional[bool] = None,
                   attn_splits: Optional[int] = None, use_mega: Optional[bool] = None, prefill_min_rows: Optional[int] = None,
                   wait_budget_ms: Optional[int] = None) -> "B200Runtime":
        lib = load_library()
        cfg = Config()
        lib.lum_config_default(C.byref(cfg))
        cfg.device = device
        if use_graph is not None:
            cfg.use_graph = int(use_graph)
        if use_pdl is not None:
            cfg.use_pdl = int(use_pdl)
        if attn_splits is not None:
            cfg.attn_splits = int(attn_splits)
        if use_mega is not None:
            cfg.use_mega = int(use_mega)
        if prefill_min_rows is not None:
            cfg.prefill_min_rows = int(prefill_min_rows)
        if wait_budget_ms is not None:
            cfg.wait_budget_ms = int(wait_budget_ms)
        h = C.c_void_p()
        rc = lib.lum_create(C.byref(cfg), C.byref(h))
        if rc != 0:
            raise LumError(rc, (lib.lum_last_error(None) or b"").decode())
        return cls(h.value, lib)

    def close(self) -> None:
        if self._h:
            self._lib.lum_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc: int) -> None:
        if rc != 0:
            raise LumError(rc, (self._lib.lum_last_error(self._h) or b"").decode())

    # ---- tensor parallel ---------------------------------------------------------------------------
    @staticmethod
    def tp_unique_id() -> bytes:
        lib = load_library()
        buf = (C.c_uint8 * 128)()
        rc = lib.lum_tp_unique_id(buf)
        if rc != 0:
            raise LumError(rc, (lib.lum_last_error(None) or b"").decode())
        return bytes(buf)

    def tp_init(self, unique_id: bytes, tp_size: int, tp_rank: int) -> None:
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        self._ck(self._lib.lum_tp_init(self._h, buf, tp_size, tp_rank))

    def tp_peer_export(self) -> bytes:
        """This rank's 64-byte IPC handle of its partial-sum exchange buffer (after ``load_model``)."""
        buf = (C.c_uint8 * 64)()
        self._ck(self._lib.lum_tp_peer_export(self._h, buf))
        return bytes(buf)

    def tp_peer_import(self, handles: Sequence[bytes]) -> None:
        """All ranks' handles in rank order: switches the K-sharded projections to the fused peer-memory exchange."""
        raw = b"".join(handles)
        buf = (C.c_uint8 * len(raw)).from_buffer_copy(raw)
        self._ck(self._lib.lum_tp_peer_import(self._h, buf, len(handles)))

    def device_info(self):
        sm, mem, cc = C.c_int32(), C.c_uint64(), C.c_int32()
        self._ck(self._lib.lum_device_info(self._h, C.byref(sm), C.byref(mem), C.byref(cc)))
        return {"sm_count": sm.value, "mem_bytes": mem.value, "cc": cc.value}

    # ---- model -----------------------------------------------------------------------------------
    def load_model(self, desc: ModelDesc) -> None:
        self._ck(self._lib.lum_model_init(self._h, C.byref(desc)))
        self.desc = desc.copy()

    def load_llir(self, blob: bytes, max_seq: int = 4096, kv_dtype: str = "bf16", max_new_tokens: int = 4096) -> None:
        """``Runtime::load_llir`` (src/op.rs:16): recognise the decoder a serialised graph describes and set it up."""
        buf = C.create_string_buffer(blob, len(blob))
        try:
            d, tok, pos, out = describe_llir(blob)
        except LumError:
            # not a decoder: a graph of primitive ops runs node by node (anything else is refused by the library, with the reason)
            self._ck(self._lib.lum_load_llir(self._h, buf, len(blob), max_seq, DTYPE[kv_dtype], max_new_tokens))
            self.desc = None
            return
        self._ck(self._lib.lum_load_llir(self._h, buf, len(blob), max_seq, DTYPE[kv_dtype], max_new_tokens))
        self.desc = d.copy(max_seq=max_seq, kv_dtype=DTYPE[kv_dtype], max_new_tokens=max_new_tokens)
        self.token_input, self.pos_input, self.logits_output = tok, pos, out

    def set_input(self, hlir_node: int, data, dtype: str) -> None:
        """``set_data(node_id, data)`` (crates/luminal_cuda/src/runtime.rs:160-165) by HLIR node id of an Input."""
        self._ck(self._lib.lum_set_input(self._h, hlir_node, data.ctypes.data_as(C.c_void_p), data.nbytes, DTYPE[dtype]))

    def set_input_device_ptr(self, hlir_node: int, device_ptr: int, nbytes: int, dtype: str) -> None:
        """``set_data`` with ``CudaInput::Ptr`` (crates/luminal_cuda/src/runtime.rs:36-39): the bytes are already on the device."""
        self._ck(self._lib.lum_set_input_device_ptr(self._h, hlir_node, C.c_void_p(device_ptr), nbytes, DTYPE[dtype]))

    def allocate_dummy_input(self, hlir_node: int, n_elems: int) -> None:
        """``Runtime::allocate_dummy_input`` (src/op.rs:24-27)."""
        self._ck(self._lib.lum_alloc_dummy_input(self._h, hlir_node, n_elems))

    def clear_intermediate_buffers(self) -> None:
        """``Runtime::clear_intermediate_buffers`` (src/op.rs:28-29)."""
        self._ck(self._lib.lum_clear_intermediates(self._h))

    def profile_llir(self, blob: bytes, dyn_map: Optional[Dict[str, int]] = None, trials: int = 4):
        """``Runtime::profile(&LLIRGraph, &dyn_map, trials)`` (src/op.rs:18-23): ``(usec per execute, display string)`` for a
        whole decoder or a chunk of layers, timed on a scratch runtime with stand-in weights."""
        dm = dyn_map or {}
        us = C.c_double()
        text = C.create_string_buffer(160)
        buf = C.create_string_buffer(blob, len(blob))
        self._ck(self._lib.lum_profile_llir(self._h, buf, len(blob), int(dm.get("s", 1)), int(dm.get("p", 0)), trials, C.byref(us), text, 160))
        return us.value, text.value.decode()

    def kv_save(self, layer: int, kind: str, rows: int):
        """Rows [0, rows) of one layer's K or V cache as raw bytes in the cache's own element type."""
        import numpy as np
        d = self.desc
        esz = 2 if d.kv_dtype == DTYPE["bf16"] else 4
        out = np.empty(rows * (d.n_kv_heads // max(1, d.tp_size)) * d.head_dim * esz, dtype=np.uint8)
        self._ck(self._lib.lum_kv_save(self._h, layer, 0 if kind == "k" else 1, rows, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def kv_load(self, layer: int, kind: str, rows: int, data) -> None:
        self._ck(self._lib.lum_kv_load(self._h, layer, 0 if kind == "k" else 1, rows, data.ctypes.data_as(C.c_void_p), data.nbytes))

    def debug_wait_timeout(self) -> None:
        """Test hook: one bounded wait runs out (raises LumError with code LUM_E_DEVICE); the runtime stays usable."""
        self._ck(self._lib.lum_debug_wait_timeout(self._h))

    def stats(self) -> Stats:
        st = Stats()
        self._ck(self._lib.lum_get_stats(self._h, C.byref(st)))
        return st

    def get_output(self, hlir_node: int):
        """``get_f32(node_id)`` (crates/luminal_cuda/src/runtime.rs:168-204) for the graph's Output: last-row logits."""
        import numpy as np
        if self.desc is None:       # a graph of primitive ops: whatever the Output holds, as f32
            n = C.c_size_t()
            self._ck(self._lib.lum_get_output_raw(self._h, hlir_node, None, 0, None, C.byref(n)))
            out = np.empty(n.value, dtype=np.float32)
        else:
            out = np.empty(self.desc.vocab, dtype=np.float32)
        self._ck(self._lib.lum_get_output(self._h, hlir_node, out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out

    def get_output_raw(self, hlir_node: int):
        """The result an Output of a primitive graph names, in its own element type: float32 / int32 / uint8 (Bool) arrays, and
        uint16 bit patterns for f16 / bf16.  Returns ``(dtype_name, array)``."""
        import numpy as np
        dt, n = C.c_uint32(), C.c_size_t()
        self._ck(self._lib.lum_get_output_raw(self._h, hlir_node, None, 0, C.byref(dt), C.byref(n)))
        name = {v: k for k, v in DTYPE.items()}[dt.value]
        out = np.empty(n.value, dtype={"f32": np.float32, "int": np.int32, "bool": np.uint8, "f16": np.uint16, "bf16": np.uint16}[name])
        self._ck(self._lib.lum_get_output_raw(self._h, hlir_node, out.ctypes.data_as(C.c_void_p), out.nbytes, None, None))
        return name, out

    def set_weight(self, slot: str, layer: int, data, dtype: str) -> None:
        """``data``: a C-contiguous numpy array holding f32 values, bf16 bit patterns (uint16) or Q8_0 wire blocks (uint8)."""
        self._ck(self._lib.lum_model_set_weight(self._h, SLOT[slot], layer, data.ctypes.data_as(C.c_void_p), data.nbytes, DTYPE[dtype]))

    def set_weight_shard(self, slot: str, layer: int, data, dtype: str) -> None:
        """As set_weight, for data that already is this rank's shard."""
        self._ck(self._lib.lum_model_set_weight_shard(self._h, SLOT[slot], layer, data.ctypes.data_as(C.c_void_p), data.nbytes, DTYPE[dtype]))

    def load_safetensors(self, path: str):
        """``load_safetensors(cx, path)`` (crates/luminal_cuda/src/runtime.rs:133-158); returns (tensors stored, tensors skipped)."""
        a, b = C.c_int32(), C.c_int32()
        self._ck(self._lib.lum_load_safetensors(self._h, path.encode(), C.byref(a), C.byref(b)))
        return a.value, b.value

    def save_safetensors(self, path: str) -> None:
        """Write this rank's shard of the weights (Q8_0 as wire blocks) to a safetensors file load_safetensors takes back."""
        self._ck(self._lib.lum_save_safetensors(self._h, path.encode()))

    def synth(self, seed: int) -> None:
        self._ck(self._lib.lum_model_synth(self._h, C.c_uint64(seed)))

    def get_weight_f32(self, slot: str, layer: int, offset: int, n: int):
        import numpy as np
        out = np.empty(n, dtype=np.float32)
        self._ck(self._lib.lum_model_get_weight_f32(self._h, SLOT[slot], layer, offset, n, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def weight_bytes(self) -> int:
        b = C.c_uint64()
        self._ck(self._lib.lum_model_weight_bytes(self._h, C.byref(b)))
        return b.value

    def kv_reset(self) -> None:
        self._ck(self._lib.lum_kv_reset(self._h))

    def kv_read(self, layer: int, kind: str, rows: int):
        import numpy as np
        d = self.desc
        out = np.empty((rows, (d.n_kv_heads // max(1, d.tp_size)) * d.head_dim), dtype=np.float32)
        self._ck(self._lib.lum_kv_read(self._h, layer, 0 if kind == "k" else 1, rows, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    # ---- the reference's decode-loop surface -------------------------------------------------------
    def set_dim(self, dim: str, value: int) -> None:
        self._ck(self._lib.lum_set_dim(self._h, dim.encode()[0:1], value))

    def set_data(self, token_ids: Sequence[int]) -> None:
        arr = (C.c_int32 * len(token_ids))(*[int(t) for t in token_ids])
        self._ck(self._lib.lum_set_tokens(self._h, arr, len(token_ids)))

    def execute(self, dyn_map: Optional[Dict[str, int]] = None) -> None:
        for k, v in (dyn_map or {}).items():
            self.set_dim(k, v)
        self._ck(self._lib.lum_execute(self._h))

    def get_f32(self):
        """Logits of the last executed row (``get_f32(logits.id)`` then taking the last row in the reference)."""
        import numpy as np
        n = self.desc.vocab // max(1, self.desc.tp_size)
        out = np.empty(n, dtype=np.float32)
        self._ck(self._lib.lum_get_logits(self._h, out.ctypes.data_as(C.POINTER(C.c_float)), n))
        return out

    def get_token(self) -> int:
        t = C.c_int32()
        self._ck(self._lib.lum_get_token(self._h, C.byref(t)))
        return t.value

    def decode_greedy(self, n_steps: int) -> None:
        self._ck(self._lib.lum_decode_greedy(self._h, n_steps))

    def decode_reset(self) -> None:
        self._ck(self._lib.lum_decode_reset(self._h))

    def get_decoded(self, n: int):
        import numpy as np
        out = np.empty(n, dtype=np.int32)
        self._ck(self._lib.lum_get_decoded(self._h, out.ctypes.data_as(C.POINTER(C.c_int32)), n))
        return out

    def synchronize(self) -> None:
        self._ck(self._lib.lum_synchronize(self._h))

    # ---- several sequences ---------------------------------------------------------------------------
    def seq_select(self, seq: int) -> None:
        """Which of the ``max_batch`` sequences ``execute`` / ``decode_greedy`` / ``kv_*`` address."""
        self._ck(self._lib.lum_seq_select(self._h, seq))

    def batch_begin(self, tokens: Sequence[int], positions: Sequence[int]) -> None:
        n = len(tokens)
        t = (C.c_int32 * n)(*[int(v) for v in tokens])
        p = (C.c_int32 * n)(*[int(v) for v in positions])
        self._ck(self._lib.lum_batch_begin(self._h, n, t, p))
        self._batch_n = n

    def batch_begin_slots(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int]) -> None:
        """Row i of the batch works on cache slot ``slots[i]`` (distinct): the hook of a continuous-batching loop."""
        n = len(tokens)
        if len(slots) != n or len(positions) != n:
            raise ValueError("slots, tokens and positions must have one entry per row")
        sl = (C.c_int32 * n)(*[int(v) for v in slots])
        t = (C.c_int32 * n)(*[int(v) for v in tokens])
        p = (C.c_int32 * n)(*[int(v) for v in positions])
        self._ck(self._lib.lum_batch_begin_slots(self._h, n, sl, t, p))
        self._batch_n = n

    def kv_copy(self, src_seq: int, dst_seq: int, rows: int) -> None:
        """The first ``rows`` cache rows of every layer copied from one sequence's slot to another's (a shared prompt prefix)."""
        self._ck(self._lib.lum_kv_copy(self._h, src_seq, dst_seq, rows))

    def kv_release(self, seq: int) -> None:
        """Paged cache: the pages of sequence ``seq`` go back to the pool (nothing to do for a contiguous cache)."""
        self._ck(self._lib.lum_kv_release(self._h, seq))

    def kv_pool(self):
        """(pages in the pool, pages free, rows per page); zeros for a contiguous cache."""
        a, b, c = C.c_int32(), C.c_int32(), C.c_int32()
        self._ck(self._lib.lum_kv_pool(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    def set_sampling(self, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0) -> None:
        """The sampler after the vocabulary projection: temperature 0 (or top_k 1) = the reference's greedy ``sample``;
        otherwise a temperature / top-k / top-p draw made on the device, a function of (logits, seed, sequence, position)."""
        if temperature <= 0.0:
            self._ck(self._lib.lum_set_sampling(self._h, None))
        else:
            s = Sampling(temperature=temperature, top_p=top_p, top_k=top_k, reserved=0, seed=seed)
            self._ck(self._lib.lum_set_sampling(self._h, C.byref(s)))

    def batch_decode(self, n_steps: int) -> None:
        self._ck(self._lib.lum_batch_decode(self._h, n_steps))

    def batch_get_decoded(self, n_steps: int):
        import numpy as np
        out = np.empty((n_steps, self._batch_n), dtype=np.int32)
        self._ck(self._lib.lum_batch_get_decoded(self._h, out.ctypes.data_as(C.POINTER(C.c_int32)), n_steps))
        return out

    def batch_get_logits(self, seq: int):
        import numpy as np
        out = np.empty(self.desc.vocab, dtype=np.float32)
        self._ck(self._lib.lum_batch_get_logits(self._h, seq, out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out

    def profile(self, trials: int = 16):
        us = C.c_double()
        buf = C.create_string_buffer(128)
        self._ck(self._lib.lum_profile(self._h, trials, C.byref(us), buf, 128))
        return us.value, buf.value.decode()

    def launches_per_step(self) -> int:
        n = C.c_int32()
        self._ck(self._lib.lum_launches_per_step(self._h, C.byref(n)))
        return n.value

    def stream(self) -> int:
        return self._lib.lum_stream(self._h) or 0

    # convenience: the reference's whole loop (examples/llama/src/main.rs:82-118), greedy
    def generate(self, prompt: Iterable[int], n_new: int):
        prompt = list(prompt)
        self.kv_reset()
        self.decode_reset()
        self.set_data(prompt)
        self.execute({"s": len(prompt), "p": 0})
        first = self.get_token()
        if n_new <= 1:
            return [first][:n_new]
        self.decode_greedy(n_new - 1)
        rest = self.get_decoded(n_new - 1)
        return [first] + [int(t) for t in rest]
