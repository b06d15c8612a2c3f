"""The fused decode step for callers that have no scratch memory to give.

Some consumers of the library cannot serve diopiRequireBuffer/diopiRequireTensor: a serving engine that
handed all free HBM to its KV pool at start-up has no allocator behind its context, and a bare C harness
may implement only the tensor accessors. diopiTokenDecodeAttentionInferenceNoAlloc runs the same kernels
on an 8 MiB array built into the library, so it must (a) give the ordinary entry point's result, (b) never
call back into the context for memory, (c) keep doing so when the array still holds the previous call's
partials, and (d) refuse problems that do not fit. Collected last on purpose: a run that stops at the first
failure has then already run every other test."""
import pytest
import torch

from oracle import golden

pytestmark = pytest.mark.gpu


def make_case(B, H, D, lens, seed, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    lens = torch.tensor(lens)
    total = int(lens.sum())
    slots = total + 9
    mx = int(lens.max())
    b_loc = torch.zeros(B, mx, dtype=torch.int32)
    start = torch.zeros(B, dtype=torch.int32)
    perm = torch.randperm(slots, generator=g)
    acc = 0
    for i in range(B):
        L = int(lens[i])
        b_loc[i, mx - L:] = perm[acc:acc + L].to(torch.int32)
        start[i] = acc
        acc += L
    dev = lambda t: t.cuda()
    return dict(q=dev(torch.randn(B, H, D, generator=g).to(dtype)), k=dev((torch.randn(slots, H, D, generator=g) * 0.6).to(dtype)),
                v=dev(torch.randn(slots, H, D, generator=g).to(dtype)), b_loc=dev(b_loc), start=dev(start), lens=dev(lens.to(torch.int32)), mx=mx)


def test_no_alloc_entry_matches_the_ordinary_one(built_libs):
    assert torch.cuda.is_available()
    from diopi_b200 import functions as F
    from diopi_b200.runtime import Context, DiopiError

    ctx = Context()
    # two different problems back to back: the second one finds the first one's partials in the array
    cases = [make_case(5, 32, 128, [700, 0, 33, 1500, 256], seed=1), make_case(3, 8, 64, [90, 411, 7], seed=2, dtype=torch.float32),
             make_case(5, 32, 128, [64, 900, 1, 300, 1200], seed=3)]
    for c in cases:
        want = torch.empty_like(c["q"])
        F.token_decode_attention(c["q"], c["k"], c["v"], want, c["b_loc"], c["start"], c["lens"], c["mx"], ctx=ctx)
        ctx.release()
        before = ctx.stats()["require_calls"]
        for _ in range(2):  # and the same problem twice in a row
            got = torch.full_like(c["q"], 5.0)
            F.token_decode_attention_noalloc(c["q"], c["k"], c["v"], got, c["b_loc"], c["start"], c["lens"], c["mx"], ctx=ctx)
            ctx.synchronize()
            tol = dict(rtol=1e-3, atol=1e-3) if c["q"].dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
            torch.testing.assert_close(got.float(), want.float(), **tol)
            assert torch.equal(got, want)  # same kernels, same partition: identical bits
        # and against the CPU oracle evaluated with fp32 accumulation, not only against the sibling entry point
        ref = golden.token_decode_attention(c["q"].cpu(), c["k"].cpu(), c["v"].cpu(), torch.zeros(c["q"].shape), c["b_loc"].cpu(),
                                            c["start"].cpu(), c["lens"].cpu(), c["mx"], upcast=True)
        torch.testing.assert_close(got.cpu().float(), ref.float(), **tol)
        assert ctx.stats()["require_calls"] == before, "the no-alloc entry point asked the context for memory"

    # a problem whose partials exceed the built-in array is refused with both numbers in the message
    big = make_case(700, 32, 128, [2] * 700, seed=4)
    out = torch.empty_like(big["q"])
    with pytest.raises(DiopiError, match="built-in array holds 8388608"):
        F.token_decode_attention_noalloc(big["q"], big["k"], big["v"], out, big["b_loc"], big["start"], big["lens"], big["mx"], ctx=ctx)
    # the ordinary entry point still serves it
    F.token_decode_attention(big["q"], big["k"], big["v"], out, big["b_loc"], big["start"], big["lens"], big["mx"], ctx=ctx)
    ctx.synchronize()
