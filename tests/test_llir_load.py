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
