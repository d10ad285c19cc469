"""`Runtime::load_llir` for serialised graphs (include/lum_llir.h): recognition of the decoder pattern on the host,
error behaviour for graphs of another shape, and — on a GPU — that a runtime set up from a graph and fed through
`set_input(node id, …)` computes what the model-plan path computes."""
import struct

import numpy as np
import pytest


@pytest.fixture(scope="module")
def L(pkg):
    from oneiron_luminal_b200 import llir
    pkg.load_library()
    return llir


FIELDS = ["n_layers", "hidden", "n_q_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "weight_dtype", "embed_dtype",
          "qk_norm", "tied_head", "rope_style"]


@pytest.mark.parametrize("name", ["tiny_f32", "small_q8", "llama3_8b_q8", "llama3_8b_q8_2layer"])
@pytest.mark.parametrize("shuffle", [False, True])
def test_describe_recovers_hyperparameters(pkg, L, name, shuffle):
    want = pkg.CONFIGS[name]
    blob, ids = L.build_llama_llir(want, shuffle_qkv=shuffle)
    got, tok, pos, out = pkg.describe_llir(blob)
    for f in FIELDS:
        assert getattr(got, f) == getattr(want, f), f
    assert abs(got.rms_eps - want.rms_eps) < 1e-12 and abs(got.rope_theta - want.rope_theta) < 1e-3
    assert (tok, pos, out) == (ids["tokens"], ids["positions"], ids["logits"])


def test_describe_variants(pkg, L):
    base = pkg.CONFIGS["small_q8"]
    d, *_ = pkg.describe_llir(L.build_llama_llir(base.copy(tied_head=1, embed_dtype=pkg.DTYPE["q8_0"]))[0])
    assert d.tied_head == 1
    d, *_ = pkg.describe_llir(L.build_llama_llir(base.copy(qk_norm=1, rope_style=1))[0])
    assert d.qk_norm == 1 and d.rope_style == 1


def test_malformed_blobs_are_refused(pkg, L):
    blob, _ = L.build_llama_llir(pkg.CONFIGS["tiny_f32"])
    for bad, what in [(b"", "truncated"), (b"\0" * 12, "magic"), (blob[:len(blob) // 2], "truncated"),
                      (blob[:4] + struct.pack("<I", 9) + blob[8:], "version")]:
        with pytest.raises(pkg.LumError, match=what):
            pkg.describe_llir(bad)
    # forward reference: node 0 takes node 5 as input
    b = L.LLIRBuilder()
    b.add("Sqrt", L.elist([4]), L.inp(5), L.elist([1]), L.elist([1]))
    with pytest.raises(pkg.LumError, match="toposorted"):
        pkg.describe_llir(b.blob())


def test_other_graphs_are_refused_with_the_node_named(pkg, L):
    b = L.LLIRBuilder()
    a = b.input(0, "a", L.F32)
    b.output(b.unary("Exp2", [8], a, [1]), 3)
    with pytest.raises(pkg.LumError, match="no RowEmbed"):
        pkg.describe_llir(b.blob())
    # a decoder whose MLP lacks the up projection
    d = pkg.CONFIGS["tiny_f32"]
    b = L.LLIRBuilder()
    tok, emb, g = b.input(0, "input", L.INT), b.input(1, "embed", L.F32), b.input(2, "g", L.F32)
    x = b.add("RowEmbed", L.elist(["s"]), L.inp(tok), L.elist([1]), L.inp(emb), L.elist([d.hidden]), L.expr(d.hidden))
    n = b.add("RowRMSNorm", L.elist(["s"]), L.inp(x), L.elist([d.hidden]), L.expr(d.hidden), L.inp(g))
    b.output(n, 9)
    with pytest.raises(pkg.LumError, match=r"node \d+ \(RowRMSNorm\)"):
        pkg.describe_llir(b.blob())


# ---------------------------------------------------------------------------------------------------------
def _host_weights(o, desc, seed):
    """Every tensor of the synthetic model as the host would hold it, keyed like build_llama_llir's ids."""
    import oracle
    return oracle.host_tensors(o, desc, seed)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["tiny_f32", "small_q8"])
def test_llir_loaded_runtime_equals_model_plan(pkg, L, oracle_lib, name):
    import oracle
    want = pkg.CONFIGS[name]
    seed, prompt = 11, [3, 1, 4, 1, 5, 9, 2, 6]
    ref = pkg.B200Runtime.initialize(device=0)
    ref.load_model(want); ref.synth(seed)
    ref.set_data(prompt); ref.execute({"s": len(prompt), "p": 0})
    ref_logits, ref_tok = ref.get_f32(), ref.get_token()
    ref.decode_greedy(8)
    ref_seq = ref.get_decoded(8)
    ref.close()

    blob, ids = L.build_llama_llir(want, shuffle_qkv=True)
    rt = pkg.B200Runtime.initialize(device=0)
    kv = {0: "f32", 2: "bf16"}[want.kv_dtype]
    rt.load_llir(blob, max_seq=want.max_seq, kv_dtype=kv, max_new_tokens=want.max_new_tokens)
    for key, (arr, dt) in oracle.host_tensors(oracle_lib, want, seed).items():
        rt.set_input(ids[key], arr, dt)
    rt.set_dim("s", len(prompt)); rt.set_dim("p", 0)
    rt.set_input(ids["tokens"], np.asarray(prompt, dtype=np.int32), "int")
    rt.set_input(ids["positions"], np.arange(len(prompt), dtype=np.int32), "int")
    rt.execute()
    logits = rt.get_output(ids["logits"])
    assert np.array_equal(logits, ref_logits)
    assert rt.get_token() == ref_tok
    rt.decode_greedy(8)
    assert np.array_equal(rt.get_decoded(8), ref_seq)
    with pytest.raises(pkg.LumError, match="not an Input"):
        rt.set_input(123456, np.zeros(4, dtype=np.float32), "f32")
    with pytest.raises(pkg.LumError, match="position ids"):
        rt.set_input(ids["positions"], np.asarray([5, 6], dtype=np.int32), "int")
    rt.close()


# --------------------------------------------------------------------------------------------------------- chunks
def test_chunk_is_recognised_on_the_host(pkg, L):
    """A chunk of layers (what the reference's search profiles, src/graph.rs:351-352) is described by its own entry and
    refused, with a message that says why, where a whole decoder is expected."""
    want = pkg.CONFIGS["small_q8"]
    blob, ids = L.build_llama_chunk_llir(want, n_layers=1)
    d, hin, hout = pkg.describe_llir_chunk(blob)
    assert (d.n_layers, d.hidden, d.n_q_heads, d.n_kv_heads, d.head_dim, d.ffn) == (1, want.hidden, want.n_q_heads, want.n_kv_heads, want.head_dim, want.ffn)
    assert (hin, hout) == (ids["hidden_in"], ids["hidden_out"]) and d.vocab == 0
    blob2, _ = L.build_llama_chunk_llir(want, n_layers=2)
    assert pkg.describe_llir_chunk(blob2)[0].n_layers == 2
    with pytest.raises(pkg.LumError, match="chunk of layers"):
        pkg.describe_llir(blob)
    whole, _ = L.build_llama_llir(want)
    with pytest.raises(pkg.LumError, match="whole decoder"):
        pkg.describe_llir_chunk(whole)


@pytest.mark.gpu
def test_search_surface_dummy_profile_clear_load_execute(pkg, L, oracle_lib):
    """The order `Graph::search` drives a runtime in (src/graph.rs:293-302, 337, 351-352, 420-424, 569-570): dummy inputs,
    profile of a chunk and of the whole graph, clear, load the stitched graph, then real data and execute."""
    import oracle
    want = pkg.CONFIGS["small_q8"]
    whole, ids = L.build_llama_llir(want)
    chunk, _ = L.build_llama_chunk_llir(want, n_layers=1)
    rt = pkg.B200Runtime.initialize(device=0)
    n_embed = want.vocab * want.hidden
    rt.allocate_dummy_input(ids["embed"], n_embed)             # before any graph: remembered
    us_c, text_c = rt.profile_llir(chunk, {"s": 1, "p": 16}, trials=3)
    us_w, text_w = rt.profile_llir(whole, {"s": 1, "p": 16}, trials=3)
    assert us_c > 0 and "chunk" in text_c and us_w > us_c and "whole decoder" in text_w
    with pytest.raises(pkg.LumError, match="chunk of layers"):
        rt.load_llir(chunk, max_seq=want.max_seq)
    rt.clear_intermediate_buffers()
    rt.load_llir(whole, max_seq=want.max_seq, kv_dtype="bf16", max_new_tokens=64)
    rt.allocate_dummy_input(ids[("q", 0)], want.n_q_heads * want.head_dim * want.hidden)
    with pytest.raises(pkg.LumError, match="elements"):
        rt.allocate_dummy_input(ids[("q", 0)], 17)
    rt.allocate_dummy_input(ids["tokens"], 4)
    rt.set_dim("p", 0)
    rt.execute()                                               # runs on stand-in contents without error
    rt.synchronize()
    rt.clear_intermediate_buffers()
    # real data, as after the search: equals the plan-loaded runtime bit for bit
    seed, prompt = 5, [9, 8, 7, 6, 5]
    for key, (arr, dt) in oracle.host_tensors(oracle_lib, want, seed).items():
        rt.set_input(ids[key], arr, dt)
    rt.set_dim("s", len(prompt)); rt.set_dim("p", 0)
    rt.set_input(ids["tokens"], np.asarray(prompt, dtype=np.int32), "int")
    rt.execute()
    got = rt.get_output(ids["logits"])
    ref = pkg.B200Runtime.initialize(device=0)
    ref.load_model(want); ref.synth(seed)
    ref.set_data(prompt); ref.execute({"s": len(prompt), "p": 0})
    assert np.array_equal(got, ref.get_f32())
    st = rt.stats()
    assert st.tokens_executed >= 4 + len(prompt) and st.kernel_launches > 0 and st.weight_bytes_per_token == ref.weight_bytes()
    assert st.last_profile_usec == pytest.approx(us_w)
    assert 0 < pkg.mbu(st, us_w, 16, 6540.8) < 1.5
    ref.close(); rt.close()


@pytest.mark.gpu
def test_device_pointer_inputs_and_kv_save_load(pkg, L, oracle_lib):
    """`CudaInput::Ptr` inputs (weights already on the device) and parking / restoring the cache."""
    import oracle
    import torch
    want = pkg.CONFIGS["small_q8"]
    blob, ids = L.build_llama_llir(want)
    seed, prompt = 21, [1, 2, 3, 4, 5, 6, 7]
    rt = pkg.B200Runtime.initialize(device=0)
    rt.load_llir(blob, max_seq=want.max_seq, kv_dtype="bf16", max_new_tokens=64)
    keep = []
    for key, (arr, dt) in oracle.host_tensors(oracle_lib, want, seed).items():
        t = torch.from_numpy(arr).cuda()
        keep.append(t)
        rt.set_input_device_ptr(ids[key], t.data_ptr(), arr.nbytes, dt)
    torch.cuda.synchronize()
    toks = torch.tensor(prompt, dtype=torch.int32, device="cuda")
    rt.set_dim("s", len(prompt)); rt.set_dim("p", 0)
    rt.set_input_device_ptr(ids["tokens"], toks.data_ptr(), 4 * len(prompt), "int")
    rt.execute()
    first = rt.get_token()
    ref = pkg.B200Runtime.initialize(device=0)
    ref.load_model(want); ref.synth(seed)
    ref.set_data(prompt); ref.execute({"s": len(prompt), "p": 0})
    assert first == ref.get_token() and np.array_equal(rt.get_f32(), ref.get_f32())
    # park the cache, wipe it, bring it back: decoding continues as if nothing happened
    rows = len(prompt)
    saved = [(l, k, rt.kv_save(l, k, rows)) for l in range(want.n_layers) for k in ("k", "v")]
    ref.decode_greedy(6)
    want_seq = ref.get_decoded(6)
    rt.kv_reset()
    for l, k, data in saved:
        rt.kv_load(l, k, rows, data)
    with pytest.raises(pkg.LumError, match="bytes"):
        rt.kv_load(0, "k", rows, saved[0][2][:-2])
    rt.set_dim("p", rows)
    rt.decode_reset()
    rt.decode_greedy(6)
    assert np.array_equal(rt.get_decoded(6), want_seq)
    ref.close(); rt.close()
