"""Weight ingest: the safetensors container, the Q8_0 quantiser, loading a float checkpoint into a quantised plan and the
shard writer.

The reference loads safetensors through `CudaRuntime::load_safetensors` (crates/luminal_cuda/src/runtime.rs:133-158: tensors are
matched to the graph's Input labels, F32 and U8 only).  It holds no Q8_0 code, so the quantiser's oracle is a restatement of
ggml's published reference quantiser; it is pinned here with blocks worked by hand (and is otherwise unpinned by reference vectors).
"""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from oracle import OracleModel, load, q8_0_dequant, q8_0_quantize


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bfloat16 bit patterns, round to nearest even (values here are finite)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------------------------------------- CPU: oracle quantiser

def test_oracle_quantiser_hand_worked_blocks():
    # 1. a block whose largest value is 127 * 2^-3: d = 2^-3 exactly, every quant is the value / d
    q = np.arange(-16, 16, dtype=np.float32) * 8 - 1          # -129 ... 119 step 8, clipped below
    q = np.clip(q, -127, 127)
    q[0] = -127
    x = q * np.float32(0.125)
    blk = q8_0_quantize(x)[0]
    assert struct.unpack("<e", bytes(blk[:2]))[0] == 0.125
    assert np.array_equal(blk[2:].view(np.int8), q.astype(np.int8))
    # 2. all zeros: scale 0, quants 0 (the reciprocal of a zero scale is taken as 0)
    blk = q8_0_quantize(np.zeros(32, np.float32))[0]
    assert not blk.any()
    # 3. halves round away from zero: max 127 -> d = 1; 0.5 -> 1, -0.5 -> -1, 2.5 -> 3, -2.5 -> -3, 1.4999 -> 1
    x = np.zeros(32, np.float32)
    x[:6] = [127.0, 0.5, -0.5, 2.5, -2.5, 1.4999]
    blk = q8_0_quantize(x)[0]
    assert list(blk[2:8].view(np.int8)) == [127, 1, -1, 3, -3, 1]
    # 4. the stored scale is the binary16 rounding of d, the quants come from the unrounded d
    x = np.zeros(32, np.float32)
    x[0], x[1] = 1.0, 0.5
    blk = q8_0_quantize(x)[0]
    d = np.float32(1.0) / np.float32(127.0)
    assert struct.unpack("<e", bytes(blk[:2]))[0] == np.float16(d)
    idv = np.float32(1.0) / d
    assert list(blk[2:4].view(np.int8)) == [int(np.round(np.float32(1.0) * idv)), int(np.floor(np.float32(0.5) * idv + np.float32(0.5)))]
    # 5. dequantising returns values within half a step of the input, plus the binary16 rounding of the scale (127 * 2^-11 steps)
    rng = np.random.default_rng(5)
    x = rng.normal(0, 0.05, 32 * 64).astype(np.float32)
    back = q8_0_dequant(q8_0_quantize(x))
    step = np.repeat(np.abs(x.reshape(-1, 32)).max(axis=1) / 127, 32)
    assert np.all(np.abs(back - x) <= (0.5 + 127 * 2.0 ** -11) * step * 1.001 + 1e-9)


# ------------------------------------------------------------------------------------------------- CPU: container

def test_safetensors_write_then_read(pkg, tmp_path):
    rng = np.random.default_rng(1)
    tensors = {
        "model.embed_tokens.weight": ("bf16", bf16_bits(rng.normal(0, 1, (7, 5)))),
        "a.f32": ("f32", rng.normal(0, 1, (3, 4, 2)).astype(np.float32)),
        "half": ("f16", rng.normal(0, 1, 9).astype(np.float16)),
        "raw \"quoted\" \\ name": ("u8", rng.integers(0, 256, 68, dtype=np.uint8)),
        "ids": ("i32", np.arange(6, dtype=np.int32).reshape(2, 3)),
        "scalar": ("f32", np.array(3.5, dtype=np.float32)),
        "empty": ("f32", np.zeros((0, 4), np.float32)),
    }
    path = str(tmp_path / "t.safetensors")
    pkg.safetensors_write(path, tensors, {"format": "pt", "lum.tp_size": 2})
    raw = open(path, "rb").read()
    (n,) = struct.unpack("<Q", raw[:8])
    assert n % 8 == 0 and raw[8:9] == b"{"                     # header padded to 8 bytes, as the format asks
    import json
    hdr = json.loads(raw[8:8 + n])                             # any JSON reader can read what the writer wrote
    assert hdr["a.f32"] == {"dtype": "F32", "shape": [3, 4, 2], "data_offsets": hdr["a.f32"]["data_offsets"]}
    assert hdr["__metadata__"] == {"format": "pt", "lum.tp_size": "2"}
    got, meta = pkg.safetensors_read(path)
    assert meta["format"] == "pt" and meta["lum.tp_size"] == "2"
    assert list(got) == list(tensors)
    for k, (dt, a) in tensors.items():
        assert got[k][0] == dt and got[k][1].shape == a.shape and np.array_equal(got[k][1], a), k


def test_safetensors_reads_a_foreign_header(pkg, tmp_path):
    """A header as other writers make it: keys in any order, unknown keys, unknown dtypes, spaces, unicode escapes."""
    a = np.arange(12, dtype=np.float32)
    b = np.arange(4, dtype=np.int64)
    hdr = ('{ "w" : {"shape":[3,4], "extra": {"x": [1, {"y": null}]}, "data_offsets":[32,80], "dtype":"F32"},'
           ' "__metadata__": {"note": "caf\\u00e9 \\"q\\""}, "big": {"dtype":"I64","shape":[4],"data_offsets":[0,32]} }   ')
    path = str(tmp_path / "f.safetensors")
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr.encode() + b.tobytes() + a.tobytes())
    got, _ = pkg.safetensors_read(path)
    assert np.array_equal(got["w"][1], a.reshape(3, 4)) and got["w"][0] == "f32"
    assert got["big"][0] == "other" and got["big"][1].tobytes() == b.tobytes()
    lib = pkg.load_library()
    h = C.c_void_p()
    assert lib.lum_st_open(path.encode(), C.byref(h)) == 0
    assert lib.lum_st_metadata(h, b"note").decode() == 'café "q"' and lib.lum_st_metadata(h, b"absent") is None
    lib.lum_st_close(h)


@pytest.mark.parametrize("content, why", [
    (b"\x05\x00", "shorter than a header"),
    (struct.pack("<Q", 1 << 40) + b"{}", "larger than the file"),
    (struct.pack("<Q", 9) + b'{"a":{"d}', "unterminated"),
    (struct.pack("<Q", 62) + b'{"a":{"dtype":"F32","shape":[4],"data_offsets":[0,16]}}       ' + b"\0" * 8, "outside the file"),
])
def test_safetensors_malformed_files_are_refused(pkg, tmp_path, content, why):
    path = str(tmp_path / "bad.safetensors")
    open(path, "wb").write(content)
    with pytest.raises(pkg.LumError) as ei:
        pkg.safetensors_read(path)
    assert why in str(ei.value)
    with pytest.raises(pkg.LumError):
        pkg.safetensors_read(str(tmp_path / "missing.safetensors"))


# ------------------------------------------------------------------------------------------------- GPU

LABELS = {"embed": "model.embed_tokens.weight", "final_norm": "model.norm.weight", "lm_head": "lm_head.weight",
          "attn_norm": "input_layernorm.weight", "mlp_norm": "post_attention_layernorm.weight", "q": "self_attn.q_proj.weight",
          "k": "self_attn.k_proj.weight", "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight",
          "gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight"}


def float_checkpoint(desc, seed, dtype):
    """A float checkpoint of the plan's shape under the reference's labels: ``name -> (slot, layer, f32 values as stored)``."""
    rng = np.random.default_rng(seed)
    H, F, V, hd = desc.hidden, desc.ffn, desc.vocab, desc.head_dim
    qd, kvd = desc.n_q_heads * hd, desc.n_kv_heads * hd
    out = {}

    def put(name, slot, layer, shape, gain=False):
        v = (1.0 + 0.1 * rng.normal(size=shape) if gain else rng.normal(0, 0.04, shape)).astype(np.float32)
        if dtype == "bf16":
            v = bf16_to_f32(bf16_bits(v))
        elif dtype == "f16":
            v = v.astype(np.float16).astype(np.float32)
        out[name] = (slot, layer, v)

    put(LABELS["embed"], "embed", 0, (V, H))
    put(LABELS["final_norm"], "final_norm", 0, (H,), True)
    put(LABELS["lm_head"], "lm_head", 0, (V, H))
    dims = {"q": (qd, H), "k": (kvd, H), "v": (kvd, H), "o": (H, qd), "gate": (F, H), "up": (F, H), "down": (H, F)}
    for l in range(desc.n_layers):
        for s, shp in dims.items():
            put(f"model.layers.{l}.{LABELS[s]}", s, l, shp)
        put(f"model.layers.{l}.{LABELS['attn_norm']}", "attn_norm", l, (H,), True)
        put(f"model.layers.{l}.{LABELS['mlp_norm']}", "mlp_norm", l, (H,), True)
    return out


def write_checkpoint(pkg, path, ck, dtype):
    t = {}
    for name, (_, _, v) in ck.items():
        t[name] = {"f32": ("f32", v), "bf16": ("bf16", bf16_bits(v)), "f16": ("f16", v.astype(np.float16))}[dtype]
    t["model.rotary_emb.inv_freq"] = ("f32", np.ones(4, np.float32))        # a label the plan does not have: skipped
    pkg.safetensors_write(path, t, {"format": "pt"})


def oracle_from_checkpoint(pkg, desc, ck):
    """The oracle model holding what the runtime should hold: linears quantised by the oracle's quantiser, the embedding and the
    gains rounded to the plan's bf16."""
    m = OracleModel(desc)
    for name, (slot, layer, v) in ck.items():
        if slot in ("embed", "final_norm", "attn_norm", "mlp_norm"):
            m.set_weight(pkg.SLOT[slot], layer, bf16_bits(v), 2)
        else:
            m.set_weight(pkg.SLOT[slot], layer, q8_0_quantize(v), 7)
    return m


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_quantiser_matches_oracle_bit_for_bit(pkg, dtype):
    import torch
    lib = pkg.load_library()
    rng = np.random.default_rng(11)
    n = 32 * 40000
    x = (rng.normal(0, 0.05, n) * np.exp(rng.normal(0, 2, n // 32)).repeat(32)).astype(np.float32)
    x[:32] = 0.0                                            # a zero block
    x[32:64] = np.float32(1e-30)                            # a scale that underflows binary16
    x[64:96] = np.arange(32) * 0.5                          # exact halves
    x[96:128] = -x[64:96]
    if dtype == "bf16":
        x = bf16_to_f32(bf16_bits(x)); src = torch.from_numpy(bf16_bits(x).view(np.int16)).cuda()
    elif dtype == "f16":
        x = x.astype(np.float16).astype(np.float32); src = torch.from_numpy(x.astype(np.float16)).cuda()
    else:
        src = torch.from_numpy(x).cuda()
    q = torch.empty(n, dtype=torch.int8, device="cuda")
    s = torch.empty(n // 32, dtype=torch.float16, device="cuda")
    assert lib.lum_op_q8_0_quantize(src.data_ptr(), pkg.DTYPE[dtype], n, q.data_ptr(), s.data_ptr(), None) == 0, lib.lum_st_last_error()
    torch.cuda.synchronize()
    want = q8_0_quantize(x)
    assert np.array_equal(q.cpu().numpy().reshape(-1, 32), want[:, 2:].view(np.int8))
    assert np.array_equal(s.cpu().numpy().view(np.uint16), want[:, :2].copy().view(np.uint16).reshape(-1))
    assert lib.lum_op_q8_0_quantize(src.data_ptr(), pkg.DTYPE[dtype], 33, q.data_ptr(), s.data_ptr(), None) != 0
    assert lib.lum_op_q8_0_quantize(src.data_ptr(), pkg.DTYPE["q8_0"], 64, q.data_ptr(), s.data_ptr(), None) != 0


@pytest.mark.gpu
@pytest.mark.parametrize("config, dtype", [("small_q8", "bf16"), ("small_q8", "f32"), ("small_q8_odd", "f16")])
def test_float_checkpoint_loads_into_a_quantised_plan(pkg, tmp_path, config, dtype):
    """load_safetensors on a float checkpoint: the linears are quantised on the GPU, the rest converted; the runtime then holds
    exactly what the oracle's quantiser makes of the same file, and decodes the oracle's tokens."""
    desc = pkg.CONFIGS[config]
    ck = float_checkpoint(desc, 21, dtype)
    path = str(tmp_path / "model.safetensors")
    write_checkpoint(pkg, path, ck, dtype)
    orc = oracle_from_checkpoint(pkg, desc, ck)
    rt = pkg.B200Runtime.initialize(device=0)
    try:
        rt.load_model(desc)
        loaded, ignored = rt.load_safetensors(path)
        assert (loaded, ignored) == (len(ck), 1)
        for name, (slot, layer, v) in ck.items():
            have = rt.get_weight_f32(slot, layer, 0, v.size)
            want = bf16_to_f32(bf16_bits(v)).reshape(-1) if slot in ("embed", "final_norm", "attn_norm", "mlp_norm") else q8_0_dequant(q8_0_quantize(v))
            assert np.array_equal(have, want), name
        prompt = orc.synth_tokens(3, 10)
        want_toks, margins = orc.generate(prompt, 12, return_margins=True)
        got = rt.generate(prompt, 12)
        assert got == want_toks, (got, want_toks, margins)
        # the same through lum_model_set_weight with a host array, one tensor
        name = "model.layers.1.self_attn.o_proj.weight"
        v = ck[name][2]
        rt.set_weight("o", 1, {"f32": v, "f16": v.astype(np.float16), "bf16": bf16_bits(v)}[dtype], dtype)
        assert np.array_equal(rt.get_weight_f32("o", 1, 0, v.size), q8_0_dequant(q8_0_quantize(v)))
        with pytest.raises(pkg.LumError):
            rt.set_weight("o", 1, v.reshape(-1)[:-32].copy(), "f32")               # wrong size
        with pytest.raises(pkg.LumError):
            rt.set_weight("attn_norm", 0, np.zeros(desc.hidden // 32 * 34, np.uint8), "q8_0")     # blocks for an unquantised slot
    finally:
        rt.close()


@pytest.mark.gpu
@pytest.mark.parametrize("config", ["small_q8", "small_q8_odd", "small_oss"])
def test_shard_file_round_trip(pkg, tmp_path, config):
    """save_safetensors writes what the runtime holds; a fresh runtime that loads the file holds the same bytes and decodes
    the same tokens; a file from another rank is refused."""
    desc = pkg.CONFIGS[config]
    path = str(tmp_path / "shard.safetensors")
    a = pkg.B200Runtime.initialize(device=0)
    b = pkg.B200Runtime.initialize(device=0)
    try:
        a.load_model(desc); a.synth(77)
        a.save_safetensors(path)
        tensors, meta = pkg.safetensors_read(path)
        assert meta["lum.shard"] == "1" and meta["lum.tp_size"] == "1" and meta["lum.ep_size"] == "1"
        qname = "model.layers.0.self_attn.q_proj.weight"
        assert tensors[qname][0] == "u8" and tensors[qname][1].shape == (desc.n_q_heads * desc.head_dim, desc.hidden // 32 * 34)
        n = desc.n_q_heads * desc.head_dim * desc.hidden
        assert np.array_equal(q8_0_dequant(tensors[qname][1]), a.get_weight_f32("q", 0, 0, n))
        b.load_model(desc)
        loaded, ignored = b.load_safetensors(path)
        assert loaded == len(tensors) and ignored == 0
        prompt = [5, 9, 2, 7, 1, 3, 8, 4]
        assert b.generate(prompt, 16) == a.generate(prompt, 16)
        b.save_safetensors(str(tmp_path / "again.safetensors"))
        again, _ = pkg.safetensors_read(str(tmp_path / "again.safetensors"))
        assert all(np.array_equal(again[k][1], tensors[k][1]) for k in tensors)
        # a file that says it is another rank's shard
        pkg.safetensors_write(str(tmp_path / "other.safetensors"), tensors, dict(meta, **{"lum.tp_size": "2", "lum.tp_rank": "1"}))
        with pytest.raises(pkg.LumError) as ei:
            b.load_safetensors(str(tmp_path / "other.safetensors"))
        assert "rank 1/2" in str(ei.value)
        assert b.generate(prompt, 16) == a.generate(prompt, 16)              # the refused load changed nothing
    finally:
        a.close(); b.close()
