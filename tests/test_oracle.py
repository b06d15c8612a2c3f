"""The CPU oracle against the reference's own outputs (tests/golden, made by make_fixtures.py from
the unmodified golden functions) and the literal known-answer values of the reference's configs."""
import numpy as np
import pytest
import torch

from conftest import fixture_names, load_fixture
from oracle import golden

TOL = {torch.float32: dict(rtol=1e-5, atol=1e-6), torch.float64: dict(rtol=1e-5, atol=1e-6),
       torch.float16: dict(rtol=2e-3, atol=1e-3), torch.bfloat16: dict(rtol=1.6e-2, atol=1e-2)}


def close(a, b):
    torch.testing.assert_close(a.double(), b.double(), **TOL[b.dtype])


@pytest.mark.parametrize("name", fixture_names("apply_penalty_v2"))
def test_apply_penalty_v2_bit_exact(name):
    f = load_fixture(name)
    got = golden.apply_penalty_v2(f["logits"].clone(), f["presence"], f["frequency"], f["repetition"], f["ids"], f["counts"])
    assert torch.equal(got, f["out"])


@pytest.mark.parametrize("name", fixture_names("rotary_emb_v2"))
def test_rotary_emb_v2(name):
    f = load_fixture(name)
    q, k = golden.rotary_emb_v2(f["query"], f["key"], f["cos"], f["sin"], f["dim"])
    assert torch.equal(q, f["out_query"]) and torch.equal(k, f["out_key"])


@pytest.mark.parametrize("name", [n for n in fixture_names("apply_penalty") if "_v2_" not in n])
def test_apply_penalty_bit_exact(name):
    f = load_fixture(name)
    got = golden.apply_penalty(f["logits"].clone(), f["presence"], f["frequency"], f["ids"], f["counts"], f["cum"], 0)
    assert torch.equal(got, f["out"])


def test_apply_penalty_hand_computed():
    """diopi_configs.py:9274-9308, worked by hand in fp32: row 0, id 0: 0.1 - 3*0.3 - 0.1 = -0.9."""
    f = load_fixture("apply_penalty_config_f32")
    ref = f["logits"].clone()
    cum = f["cum"].tolist()
    for i in range(3):
        for e in range(cum[i], cum[i + 1]):
            t = int(f["ids"][e])
            ref[i, t] = (f["logits"][i, t] - np.float32(int(f["counts"][e])) * f["frequency"][i]) - f["presence"][i]
    assert torch.equal(ref, f["out"])
    assert abs(float(f["out"][0, 0]) + 0.9) < 1e-6


@pytest.mark.parametrize("name", fixture_names("destindex_copy_kv"))
def test_destindex_copy_kv(name):
    f = load_fixture(name)
    got = golden.destindex_copy_kv(f["k"], f["dest_loc"], f["out_before"].clone())
    assert torch.equal(got, f["out"])


def _pool(f, key):
    rows = f[key]
    pool = torch.zeros((f["pool"],) + tuple(rows.shape[1:]), dtype=rows.dtype)
    pool[f["used"].long()] = rows
    return pool


@pytest.mark.parametrize("name", fixture_names("token_attention_config"))
def test_token_attention_config(name):
    f = load_fixture(name)
    k, v = _pool(f, "k_rows"), _pool(f, "v_rows")
    H = f["q"].shape[1]
    att = golden.token_attention(f["q"], k, torch.zeros(H, 13, dtype=k.dtype), f["b_loc"], f["b_start_loc"], f["b_seq_len"], f["max_input_len"])
    close(att, f["att"])
    red = golden.token_softmax_reducev(f["logics"], v, torch.zeros_like(f["reducev"]), f["b_loc"], f["b_start_loc"], f["b_seq_len"], f["max_input_len"], 10)
    close(red, f["reducev"])
    fused = golden.token_decode_attention(f["q"], k, v, torch.zeros_like(f["fused"]), f["b_loc"], f["b_start_loc"], f["b_seq_len"], f["max_input_len"])
    close(fused, f["fused"])


@pytest.mark.parametrize("name", fixture_names("decode_seeded"))
def test_decode_seeded(name):
    f = load_fixture(name)
    att = golden.token_attention(f["q"], f["k"], torch.zeros_like(f["att"]), f["b_loc"], f["b_start_loc"], f["b_seq_len"], f["max_input_len"])
    close(att, f["att"])
    out = golden.token_softmax_reducev(f["att"], f["v"], torch.zeros_like(f["out"]), f["b_loc"], f["b_start_loc"], f["b_seq_len"], f["max_input_len"])
    close(out, f["out"])
    # the fp32-accumulation form agrees with the input-dtype form within half precision
    up = golden.token_decode_attention(f["q"], f["k"], f["v"], torch.zeros_like(f["out"]), f["b_loc"], f["b_start_loc"], f["b_seq_len"],
                                       f["max_input_len"], upcast=True)
    torch.testing.assert_close(up.float(), f["out"].float(), rtol=1e-2, atol=1e-2)
    # a request of length 0 yields zeros
    empty = (f["b_seq_len"] == 0).nonzero().flatten()
    for i in empty.tolist():
        assert torch.count_nonzero(f["out"][i]) == 0


@pytest.mark.parametrize("name", fixture_names("context_attention"))
def test_context_attention(name):
    f = load_fixture(name)
    out = golden.context_attention(f["q"], f["k"], f["v"], torch.zeros_like(f["out"]), f["b_start_loc"], f["b_seq_len"], f["max_input_len"])
    close(out, f["out"])
    blocked = golden.context_attention(f["q"], f["k"], f["v"], torch.zeros_like(f["out"]), f["b_start_loc"], f["b_seq_len"], f["max_input_len"], row_block=5)
    close(blocked, f["out"])


@pytest.mark.parametrize("name", [n for n in fixture_names("rotary_emb") if "_v2_" not in n])
def test_rotary_emb(name):
    f = load_fixture(name)
    close(golden.rotary_emb(f["x"], f["cos"], f["sin"], bool(f["conj"]), False), f["out"])
    if f["x"].dtype == torch.float64:
        torch.testing.assert_close(golden.rotary_emb_f64(f["x"], f["cos"], f["sin"], bool(f["conj"])), f["out"], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", [n for n in fixture_names("rms_norm") if "_backward_" not in n])
def test_rms_norm(name):
    f = load_fixture(name)
    got = golden.rms_norm(f["x"], tuple(f["normalized_shape"].tolist()), f["weight"], f.get("bias"), f["eps"])
    close(got, f["out"])


# tolerance of the backward fixtures: the harness's 1e-4 for fp32/fp64 (diopi_configs.py:9139-9140). In the half types
# autograd rounds the two terms of grad_input to the storage type separately and adds them there, the closed form
# rounds once: up to a few units in the last place apart (relative 2^-10 for fp16, 2^-7 for bf16).
BWD_TOL = {torch.float32: dict(rtol=1e-4, atol=1e-4), torch.float64: dict(rtol=1e-4, atol=1e-4),
           torch.float16: dict(rtol=4e-3, atol=4e-3), torch.bfloat16: dict(rtol=3e-2, atol=3e-2)}


@pytest.mark.parametrize("name", fixture_names("rms_norm_backward"))
def test_rms_norm_backward(name):
    f = load_fixture(name)
    ns = tuple(f["normalized_shape"].tolist())
    t = BWD_TOL[f["x"].dtype]
    for g, pre in ((f["grad_output"], ""), (torch.ones_like(f["x"]), "ones_")):
        dx, dw, db = golden.rms_norm_backward(g, f["x"], f["weight"], ns, eps=f["eps"], with_bias="bias" in f)
        torch.testing.assert_close(dx.double(), f[pre + "grad_input"].double(), **t)
        torch.testing.assert_close(dw.double(), f[pre + "grad_weight"].double(), **t)
        if "bias" in f:
            torch.testing.assert_close(db.double(), f[pre + "grad_bias"].double(), **t)
        else:
            assert db is None


@pytest.mark.parametrize("name", fixture_names("prompt_flash_attention"))
def test_prompt_flash_attention(name):
    f = load_fixture(name)
    bs, mlen, heads = f["batch"], f["max_input_len"], f["heads"]
    got = golden.prompt_flash_attention(f["query"], f["key"], f["value"], None, [mlen] * bs, mlen, heads, heads, 128)
    close(got, f["out"])


@pytest.mark.parametrize("name", fixture_names("paged_attention"))
def test_paged_attention(name):
    f = load_fixture(name)
    heads = f["heads"]
    got = golden.paged_attention(f["query"], f["key"], f["value"], None, [5], heads, heads, 128, torch.tensor([[0, 1]], dtype=torch.int32), 128)
    close(got, f["out"])
