"""ctypes wrapper of the CPU oracle (oracle/liblum_oracle.so).  Test infrastructure: only tests,
the smoke check and the benchmark's CPU-baseline leg import this."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB_PATH = os.path.join(ORACLE_DIR, "liblum_oracle.so")

_lib = None


class OrcCfg(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int32), ("hidden", C.c_int32), ("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32), ("max_seq", C.c_int32),
        ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("rope_style", C.c_int32), ("weight_q8", C.c_int32),
        ("kv_bf16", C.c_int32), ("embed_bf16", C.c_int32), ("qk_norm", C.c_int32), ("tied_head", C.c_int32),
        ("sliding_window", C.c_int32), ("window_even_layers", C.c_int32), ("attn_sinks", C.c_int32), ("proj_bias", C.c_int32),
        ("yarn_factor", C.c_float), ("yarn_beta_fast", C.c_float), ("yarn_beta_slow", C.c_float), ("yarn_orig_max_pos", C.c_float),
        ("n_experts", C.c_int32), ("top_k", C.c_int32), ("swiglu_limit", C.c_float),
    ]


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    srcs = [os.path.join(ORACLE_DIR, f) for f in os.listdir(ORACLE_DIR) if f.endswith((".cpp", ".hpp"))]
    if not os.path.exists(LIB_PATH) or any(os.path.getmtime(s) > os.path.getmtime(LIB_PATH) for s in srcs):
        subprocess.run(["make", "-C", ORACLE_DIR], check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, u32, u64, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_size_t
    fp, ip = C.POINTER(C.c_float), C.POINTER(C.c_int32)
    sig = {
        "orc_native_create": (vp, [vp, sz, C.c_char_p, sz]),
        "orc_native_destroy": (None, [vp]),
        "orc_native_error": (C.c_char_p, [vp]),
        "orc_native_set_dim": (i32, [vp, C.c_char, i64]),
        "orc_native_set_data": (i32, [vp, i64, vp, sz, u32]),
        "orc_native_execute": (i32, [vp]),
        "orc_native_output_len": (i64, [vp, i64]),
        "orc_native_output_dtype": (i32, [vp, i64]),
        "orc_native_get_f32": (i32, [vp, i64, fp, sz]),
        "orc_native_get_i32": (i32, [vp, i64, ip, sz]),
        "orc_model_create": (vp, [C.POINTER(OrcCfg)]),
        "orc_model_destroy": (None, [vp]),
        "orc_model_error": (C.c_char_p, [vp]),
        "orc_q8_0_dequant": (None, [vp, sz, fp]),
        "orc_q8_0_quantize": (None, [fp, sz, vp]),
        "orc_sample_topk": (i32, [fp, i32, C.c_float, i32, C.c_float, u64, i32, i32, fp]),
        "orc_synth": (i32, [u64, u64, u32, sz, i32, vp]),
        "orc_synth_range": (i32, [u64, u64, u32, sz, sz, vp]),
        "orc_synth_tokens": (None, [u64, u64, u32, sz, ip]),
        "orc_model_set_weight": (i32, [vp, i32, i32, vp, u32]),
        "orc_model_synth": (i32, [vp, u64]),
        "orc_model_forward": (i32, [vp, ip, i32, i32, fp, i32]),
        "orc_argmax_last": (i32, [fp, i32]),
        "orc_top2_margin": (C.c_float, [fp, i32]),
        "orc_model_kv_reset": (None, [vp]),
        "orc_model_kv_fill": (i32, [vp, u64, i32]),
        "orc_model_kv_read": (i32, [vp, i32, i32, i32, fp]),
        "orc_rmsnorm": (None, [fp, fp, i32, C.c_float, fp]),
        "orc_matvec_f32": (None, [fp, i32, i32, fp, fp]),
        "orc_matvec_q8_0": (None, [vp, i32, i32, fp, fp]),
        "orc_rope": (None, [fp, i32, i32, i32, C.c_float, i32]),
        "orc_swiglu": (None, [fp, fp, i32, fp]),
        "orc_round6": (C.c_float, [C.c_double]),
        "orc_f32_to_f16": (C.c_uint16, [C.c_float]),
        "orc_f16_to_f32": (C.c_float, [C.c_uint16]),
        "orc_f32_to_bf16": (C.c_uint16, [C.c_float]),
        "orc_threads": (i32, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def q8_0_quantize(x: np.ndarray) -> np.ndarray:
    """f32 values (a multiple of 32 of them) -> Q8_0 wire blocks [n / 32, 34] uint8, by the oracle's quantiser."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    assert x.size % 32 == 0
    out = np.empty((x.size // 32, 34), dtype=np.uint8)
    load().orc_q8_0_quantize(_fp(x), x.size // 32, out.ctypes.data_as(C.c_void_p))
    return out


def sample_topk(logits: np.ndarray, temperature: float, top_k: int, top_p: float, seed: int, seq: int, pos: int):
    """One draw from a row of logits by the oracle's sampler: (token, margin) — see orc_sample_topk for the margin."""
    logits = np.ascontiguousarray(logits, dtype=np.float32).reshape(-1)
    m = C.c_float(0.0)
    tok = load().orc_sample_topk(_fp(logits), logits.size, temperature, top_k, top_p, seed, seq, pos, C.byref(m))
    return int(tok), float(m.value)


def q8_0_dequant(blocks: np.ndarray) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 34)
    out = np.empty(blocks.shape[0] * 32, dtype=np.float32)
    load().orc_q8_0_dequant(blocks.ctypes.data_as(C.c_void_p), blocks.shape[0], _fp(out))
    return out


TOKENS_TID = 1 << 20  # generator id of prompt token streams


def cfg_from_desc(d) -> OrcCfg:
    """Translate the runtime's model description (lum_model_desc) into the oracle's."""
    c = OrcCfg()
    for f in ("n_layers", "hidden", "n_q_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "max_seq", "rms_eps",
              "rope_theta", "rope_style", "qk_norm", "tied_head"):
        setattr(c, f, getattr(d, f))
    for f in ("sliding_window", "window_even_layers", "attn_sinks", "proj_bias", "yarn_factor", "yarn_beta_fast", "yarn_beta_slow",
              "yarn_orig_max_pos", "n_experts", "top_k", "swiglu_limit"):
        setattr(c, f, getattr(d, f, 0))
    c.weight_q8 = 1 if d.weight_dtype == 7 else 0
    c.kv_bf16 = 1 if d.kv_dtype == 2 else 0
    c.embed_bf16 = 1 if d.embed_dtype == 2 else 0
    return c


class OracleModel:
    def __init__(self, desc):
        self.lib = load()
        self.cfg = cfg_from_desc(desc)
        self.h = C.c_void_p(self.lib.orc_model_create(C.byref(self.cfg)))

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.orc_model_destroy(self.h)
            self.h = None

    def _ck(self, rc):
        if rc != 0:
            raise RuntimeError("oracle: " + (self.lib.orc_model_error(self.h) or b"").decode())

    def synth(self, seed: int):
        self._ck(self.lib.orc_model_synth(self.h, seed))

    def set_weight(self, slot: int, layer: int, data: np.ndarray, dtype: int):
        self._ck(self.lib.orc_model_set_weight(self.h, slot, layer, data.ctypes.data_as(C.c_void_p), dtype))

    def synth_tokens(self, seed: int, n: int, stream: int = 0):
        out = np.empty(n, dtype=np.int32)
        self.lib.orc_synth_tokens(seed, TOKENS_TID + stream, self.cfg.vocab, n, out.ctypes.data_as(C.POINTER(C.c_int32)))
        return [int(t) for t in out]

    def kv_reset(self):
        self.lib.orc_model_kv_reset(self.h)

    def kv_fill(self, seed: int, rows: int):
        """Seeded stand-in contents for cache rows [0, rows) of every layer (timing runs at a long context)."""
        self._ck(self.lib.orc_model_kv_fill(self.h, seed, rows))

    def kv_read(self, layer: int, kind: str, rows: int):
        out = np.empty((rows, self.cfg.n_kv_heads * self.cfg.head_dim), dtype=np.float32)
        self._ck(self.lib.orc_model_kv_read(self.h, layer, 0 if kind == "k" else 1, rows, _fp(out)))
        return out

    def forward(self, tokens, p: int, all_rows: bool = False):
        toks = np.asarray(tokens, dtype=np.int32)
        rows = len(toks) if all_rows else 1
        out = np.empty((rows, self.cfg.vocab), dtype=np.float32)
        self._ck(self.lib.orc_model_forward(self.h, toks.ctypes.data_as(C.POINTER(C.c_int32)), len(toks), p, _fp(out), int(all_rows)))
        return out

    def argmax(self, row: np.ndarray) -> int:
        row = np.ascontiguousarray(row, dtype=np.float32)
        return int(self.lib.orc_argmax_last(_fp(row), row.size))

    def margin(self, row: np.ndarray) -> float:
        row = np.ascontiguousarray(row, dtype=np.float32)
        return float(self.lib.orc_top2_margin(_fp(row), row.size))

    def generate(self, prompt, n_new: int, return_last_logits: bool = False, return_margins: bool = False):
        """The reference's greedy loop (examples/llama/src/main.rs:82-118) on the oracle."""
        self.kv_reset()
        prompt = list(prompt)
        logits = self.forward(prompt, 0)[0]
        toks, margins = [self.argmax(logits)], [self.margin(logits)]
        p = len(prompt)
        while len(toks) < n_new:
            logits = self.forward([toks[-1]], p)[0]
            p += 1
            toks.append(self.argmax(logits))
            margins.append(self.margin(logits))
        res = [toks]
        if return_last_logits:
            res.append(logits)
        if return_margins:
            res.append(margins)
        return res[0] if len(res) == 1 else tuple(res)


def host_tensors(lib, desc, seed: int):
    """Every tensor of the synthetic model `seed` as a host would hold it before upload: ``key -> (uint8 array, dtype
    name)``, keys as in ``llir.build_llama_llir`` ("embed", "final_norm", "lm_head", (name, layer)).  Tensor ids follow
    the generator's convention: layer * 16 + slot, with the model-level tensors at layer == n_layers."""
    names = {0: "f32", 2: "bf16", 7: "q8_0"}
    slot = {"embed": 0, "attn_norm": 1, "q": 2, "k": 3, "v": 4, "o": 5, "mlp_norm": 6, "gate": 7, "up": 8, "down": 9,
            "final_norm": 10, "lm_head": 11}
    H, F, V, hd = desc.hidden, desc.ffn, desc.vocab, desc.head_dim
    qd, kvd = desc.n_q_heads * hd, desc.n_kv_heads * hd
    dims = {"q": (qd, H), "k": (kvd, H), "v": (kvd, H), "o": (H, qd), "gate": (F, H), "up": (F, H), "down": (H, F)}
    wdt, edt = desc.weight_dtype, desc.embed_dtype

    def synth(tid, dt, n, ones=0):
        size = n // 32 * 34 if dt == 7 else n * (2 if dt == 2 else 4)
        buf = np.empty(size, dtype=np.uint8)
        assert lib.orc_synth(seed, tid, dt, n, ones, buf.ctypes.data_as(C.c_void_p)) == 0
        return buf, names[dt]

    L = desc.n_layers
    out = {"embed": synth(L * 16 + 0, edt, V * H), "final_norm": synth(L * 16 + 10, edt, H, 1)}
    if not desc.tied_head:
        out["lm_head"] = synth(L * 16 + 11, wdt, V * H)
    for l in range(L):
        for name, (n, k) in dims.items():
            out[(name, l)] = synth(l * 16 + slot[name], wdt, n * k)
        out[("attn_norm", l)] = synth(l * 16 + 1, edt, H, 1)
        out[("mlp_norm", l)] = synth(l * 16 + 6, edt, H, 1)
    return out
