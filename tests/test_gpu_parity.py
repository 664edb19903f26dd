"""Parity of the CUDA kernels (called through the C ABI) with the oracle.

Error metric everywhere: max|x - ref| / max|ref| per tensor, with ref = the
fp64 oracle evaluated on the same (already rounded) inputs.
Tolerances: 1e-4 for fp32 problems, 2e-2 for bf16 problems (fp32 accumulation).
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN, ROOT, make_inputs
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-4
TOL_BF16 = 2e-2
OUT_NAMES = ("dq2", "dk2", "dv2", "ddo")


def _oracle(x64, scale, causal):
    """fp64 oracle results + saved forward tensors, all (BH, N, D).

    Causal with n_k < n_q: the first n_q - n_k queries see no key.  The oracle is evaluated on the
    remaining queries (the mask is bottom-right aligned, so that is the same problem) and the
    dead queries get zero result rows, L = -inf and O = 0, which is how the library defines them."""
    nq, nk = x64["q"].shape[1], x64["k"].shape[1]
    if causal and nk < nq:
        dead = nq - nk
        live = {n: (t[:, dead:] if n in ("q", "do", "ddq") else t) for n, t in x64.items()}
        ref, lse, o, stats = _oracle(live, scale, causal)
        z, zv = torch.zeros_like(x64["q"][:, :dead]), torch.zeros_like(x64["do"][:, :dead])   # head dims d and d_v
        ref = (torch.cat([z, ref[0]], 1), ref[1], ref[2], torch.cat([zv, ref[3]], 1))
        lse = torch.cat([torch.full((lse.shape[0], dead), -float("inf"), dtype=lse.dtype), lse], 1)
        stats = tuple(torch.cat([z[:, :, 0], t], 1) for t in stats)
        return ref, lse, torch.cat([zv, o], 1), stats
    vals = list(x64.values())
    ref = O.bwdbwd_closed_form(*vals, scale, causal)
    lse = O.attn_lse(x64["q"], x64["k"], scale, causal)
    o = O.attn_fwd(x64["q"], x64["k"], x64["v"], scale, causal)
    stats = O.bwdbwd_row_stats(*vals, scale, causal)
    return ref, lse, o, stats


def _run(x64, scale, causal, dtype, impl, upto=None, fused12=False):
    import fhob
    ref, lse, o, stats = _oracle(x64, scale, causal)
    dev = {k: v.to(dtype).cuda() for k, v in x64.items()}
    o_dev = o.to(dtype).cuda()
    lse_dev = lse.float().cuda()
    args = (dev["q"], dev["k"], dev["v"], o_dev, dev["do"], dev["ddq"], dev["ddk"], dev["ddv"], lse_dev, scale)
    if upto is None:
        got = fhob.flash_bwdbwd(*args, is_causal=causal, impl=impl, check=True)
        return got, ref, stats
    return fhob.run_passes(*args, is_causal=causal, impl=impl, upto=upto, fused12=fused12), ref, stats


SMALL = [(2, 128, 128, 64), (2, 128, 256, 64), (1, 256, 128, 128), (3, 96, 160, 32), (1, 100, 150, 72)]


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("bh,nq,nk,d", SMALL)
def test_fp32_cuda_core_path(bh, nq, nk, d, causal):
    x = make_inputs(bh, nq, nk, d, seed=21, dtype=torch.float64)
    got, ref, _ = _run(x, d ** -0.5, causal, torch.float32, "simt")
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < TOL_F32, n


FP32_TC_CASES = [(2, 128, 128, False, None), (2, 256, 384, False, None), (2, 384, 256, True, None),
                 (3, 200, 328, True, None), (1, 99, 131, False, None), (2, 320, 320, True, 70), (1, 1, 300, False, None)]


@pytest.mark.parametrize("bh,nq,nk,causal,window", FP32_TC_CASES)
def test_fp32_tensor_core_path(bh, nq, nk, causal, window):
    """fp32 problems with head dim 64 on the tensor cores: every operand as a bf16 hi + lo pair,
    three products per contraction, fp32 accumulation.  Same 1e-4 bound as the CUDA-core path,
    for the four results, the row statistics (both the two-pass and the one-sweep form) and the
    call without the saved output."""
    import fhob
    import math
    wl = math.inf if window is None else window
    x = make_inputs(bh, nq, nk, 64, seed=23, dtype=torch.float64)
    scale = 0.125
    if causal and nk < nq and window is None:
        ref, lse, o, stats = _oracle(x, scale, causal)
    else:
        ref = O.bwdbwd_closed_form(*x.values(), scale, causal, sliding_window_length=wl)
        lse = O.attn_lse(x["q"], x["k"], scale, causal, sliding_window_length=wl)
        o = O.attn_fwd(x["q"], x["k"], x["v"], scale, causal, sliding_window_length=wl)
        stats = O.bwdbwd_row_stats(*x.values(), scale, causal) if window is None else None
    dev = {k: v.float().cuda() for k, v in x.items()}
    args = (dev["q"], dev["k"], dev["v"], o.float().cuda(), dev["do"], dev["ddq"], dev["ddk"], dev["ddv"],
            lse.float().cuda(), scale)
    kw = dict(is_causal=causal, sliding_window=window, impl="tcgen05")
    got = fhob.flash_bwdbwd(*args, check=True, **kw)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert g.dtype == torch.float32 and O.rel_err(g, r) < TOL_F32, n
    again = fhob.flash_bwdbwd(*args, check=True, **kw)
    for a, b in zip(got, again):
        assert torch.equal(a, b)                      # bit-exact run to run
    auto = fhob.flash_bwdbwd(*args, check=True, **dict(kw, impl="auto"))
    for a, b in zip(got, auto):
        assert torch.equal(a, b)                      # AUTO takes the same path when the workspace has the room
    got = fhob.flash_bwdbwd(*args[:3], None, *args[4:], check=True, **kw)      # D from the sweep
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < TOL_F32, n
    if stats is not None:
        for fused in (False, True):
            res = fhob.run_passes(*args, is_causal=causal, impl="tcgen05", upto=2, fused12=fused)
            assert res["status"] == 0
            for n, r in zip(("d", "dd", "b"), stats):
                assert O.rel_err(res[n], r) < TOL_F32, (n, fused)
    # the producers either side, same scheme: forward (O and L), logsumexp alone, first backward
    live = slice(nq - nk if (causal and nk < nq) else 0, None)
    o_dev, lse_dev = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, check=True, **kw)
    assert o_dev.dtype == torch.float32
    assert O.rel_err(o_dev[:, live], o[:, live]) < TOL_F32 and O.rel_err(lse_dev[:, live], lse[:, live]) < 1e-5
    _, lse_only = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, need_o=False, **kw)
    assert O.rel_err(lse_only[:, live], lse[:, live]) < 1e-5
    first = fhob.attention_backward(dev["q"], dev["k"], dev["v"], args[3], dev["do"], args[8], scale, **kw)
    xl = {n: (t[:, live] if n in ("q", "do") else t) for n, t in x.items()}
    first_ref = O.attn_bwd(xl["q"], xl["k"], xl["v"], xl["do"], scale, causal, sliding_window_length=wl)
    assert O.rel_err(first[0][:, live], first_ref[0]) < TOL_F32
    assert O.rel_err(first[1], first_ref[1]) < TOL_F32 and O.rel_err(first[2], first_ref[2]) < TOL_F32


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("bh,nq,nk,dqk,dv", [(2, 256, 384, 32, 32), (2, 200, 328, 48, 64), (1, 320, 320, 64, 16),
                                             (2, 130, 259, 4, 60)])
def test_fp32_tensor_core_path_with_smaller_head_dims(bh, nq, nk, dqk, dv, causal):
    """fp32 with head dims below 64 (multiples of 4): the bf16 hi/lo copies are padded to 64 columns."""
    import fhob
    g = torch.Generator().manual_seed(433)
    shapes = dict(q=(bh, nq, dqk), k=(bh, nk, dqk), v=(bh, nk, dv), do=(bh, nq, dv),
                  ddq=(bh, nq, dqk), ddk=(bh, nk, dqk), ddv=(bh, nk, dv))
    x = {n: torch.randn(s, generator=g).bfloat16().double() for n, s in shapes.items()}
    scale = dqk ** -0.5
    ref = O.bwdbwd_closed_form(*x.values(), scale, causal)
    o_ref = O.attn_fwd(x["q"], x["k"], x["v"], scale, causal)
    l_ref = O.attn_lse(x["q"], x["k"], scale, causal)
    dev = {k: v.float().cuda() for k, v in x.items()}
    kw = dict(is_causal=causal, impl="tcgen05")
    got = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], o_ref.float().cuda(), dev["do"], dev["ddq"], dev["ddk"],
                            dev["ddv"], l_ref.float().cuda(), scale, check=True, **kw)
    for n, g_, r in zip(OUT_NAMES, got, ref):
        assert g_.shape == r.shape and O.rel_err(g_, r) < TOL_F32, n
    o, lse = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, check=True, **kw)
    assert o.shape == (bh, nq, dv) and O.rel_err(o, o_ref) < TOL_F32 and O.rel_err(lse, l_ref) < 1e-5
    first = fhob.attention_backward(dev["q"], dev["k"], dev["v"], o, dev["do"], lse, scale, **kw)
    first_ref = O.attn_bwd(x["q"], x["k"], x["v"], x["do"], scale, causal)
    for n, g_, r in zip(("dq", "dk", "dv"), first, first_ref):
        assert g_.shape == r.shape and O.rel_err(g_, r) < TOL_F32, n


def test_fp32_tensor_core_path_needs_head_dim_64_and_a_larger_workspace():
    import fhob
    from fhob import _lib
    import ctypes as C
    x = make_inputs(2, 128, 128, 128, seed=25, dtype=torch.float32, device="cuda")
    L = torch.zeros(2, 128, device="cuda")
    with pytest.raises(RuntimeError, match="shape not supported"):
        fhob.flash_bwdbwd(x["q"], x["k"], x["v"], x["q"], x["do"], x["ddq"], x["ddk"], x["ddv"], L, 0.1, impl="tcgen05")
    x = make_inputs(2, 128, 256, 64, seed=25, dtype=torch.float32, device="cuda")
    lib = _lib.load()
    small = torch.empty(lib.fhob_workspace_bytes(2, 128), dtype=torch.uint8, device="cuda")
    p = _lib.FhobProblem()
    p.bh, p.n_q, p.n_k, p.d, p.dtype = 2, 128, 256, 64, _lib.FHOB_F32
    assert lib.fhob_workspace_bytes_problem(C.byref(p)) >= small.numel() + (3 * 128 + 4 * 256) * 2 * 256
    with pytest.raises(RuntimeError, match="workspace"):
        fhob.flash_bwdbwd(x["q"], x["k"], x["v"], x["q"], x["do"], x["ddq"], x["ddk"], x["ddv"], L, 0.125,
                          impl="tcgen05", workspace=small)
    # AUTO with the small workspace: the CUDA-core kernels, same results to the fp32 bound
    o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], 0.125)
    args = (x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, 0.125)
    a = fhob.flash_bwdbwd(*args, workspace=small, check=True)
    b = fhob.flash_bwdbwd(*args, check=True)
    for u, v in zip(a, b):
        assert O.rel_err(u, v) < TOL_F32 and not torch.equal(u, v)      # two different kernel families


@pytest.mark.parametrize("impl", ["auto", "simt"])
def test_fp32_config_one(impl):
    """B=1 H=2 N=256 D=64 non-causal fp32, 4-D layout, against grad-of-grad (form A); `auto` runs it
    on the tensor cores (split operands), `simt` on CUDA cores."""
    import fhob
    x = make_inputs(2, 256, 256, 64, seed=1234, dtype=torch.float64)
    ref = O.bwdbwd_autograd(*x.values(), 0.125, False)
    lse = O.attn_lse(x["q"], x["k"], 0.125)
    o = O.attn_fwd(x["q"], x["k"], x["v"], 0.125)
    dev = {k: v.float().cuda().reshape(1, 2, 256, 64) for k, v in x.items()}
    got = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], o.float().cuda().reshape(1, 2, 256, 64), dev["do"],
                            dev["ddq"], dev["ddk"], dev["ddv"], lse.float().cuda().reshape(1, 2, 256), 0.125,
                            check=True, impl=impl)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert g.shape == (1, 2, 256, 64)
        assert O.rel_err(g.reshape(2, 256, 64), r) < TOL_F32, n


@pytest.mark.parametrize("upto", [1, 2])
@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
def test_bf16_row_statistics(d, causal, impl, upto):
    """Passes 1 and 2 in isolation: the dd and b row vectors."""
    x = make_inputs(2, 256, 384, d, seed=31, dtype=torch.float64)
    res, _, (sd, sdd, sb) = _run(x, d ** -0.5, causal, torch.bfloat16, impl, upto=upto)
    assert res["status"] == 0
    assert O.rel_err(res["d"], sd) < TOL_BF16
    assert O.rel_err(res["dd"], sdd) < TOL_BF16
    if upto >= 2:
        assert O.rel_err(res["b"], sb) < TOL_BF16


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
def test_bf16_row_statistics_single_sweep(d, causal, impl):
    """dd and b from the one-sweep stage (b = sum P (X + dP ddS) - 2 D dd) against the oracle and
    against the two reference-shaped passes."""
    x = make_inputs(2, 256, 384, d, seed=33, dtype=torch.float64)
    two, _, (sd, sdd, sb) = _run(x, d ** -0.5, causal, torch.bfloat16, impl, upto=2)
    one, _, _ = _run(x, d ** -0.5, causal, torch.bfloat16, impl, upto=2, fused12=True)
    assert one["status"] == 0
    assert O.rel_err(one["dd"], sdd) < TOL_BF16
    assert O.rel_err(one["b"], sb) < TOL_BF16
    assert O.rel_err(one["dd"], two["dd"]) < 1e-5
    assert O.rel_err(one["b"], two["b"]) < 5e-3


@pytest.mark.parametrize("causal", [False, True])
def test_bf16_offset_cotangents(causal):
    """Cotangents with a large common component make D and dd large against the fluctuating part of
    b: the one-sweep form of b subtracts 2 D dd from sums of that size."""
    x = make_inputs(2, 384, 384, 128, seed=35, dtype=torch.float64)
    x["do"] = x["do"] + 1.5 * x["v"].mean(dim=1, keepdim=True).sign()
    x["ddq"] = x["ddq"] + 0.75
    x["ddk"] = x["ddk"] - 0.5
    got, ref, _ = _run(x, 128 ** -0.5, causal, torch.bfloat16, "tcgen05")
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < TOL_BF16, n


BF16_CASES = [(2, 128, 128, 64), (2, 256, 384, 64), (2, 384, 256, 128), (1, 128, 512, 128), (3, 512, 512, 64)]


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("bh,nq,nk,d", BF16_CASES)
def test_bf16_outputs(bh, nq, nk, d, causal, impl):
    x = make_inputs(bh, nq, nk, d, seed=41, dtype=torch.float64)
    got, ref, _ = _run(x, d ** -0.5, causal, torch.bfloat16, impl)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert g.dtype == torch.bfloat16
        assert O.rel_err(g, r) < TOL_BF16, n


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("nq,nk,d", [(200, 328, 64), (72, 136, 128), (132, 260, 128)])
def test_bf16_ragged_lengths(nq, nk, d, causal):
    """Sequence lengths that are not multiples of the tile sizes (TMA zero fill + masking)."""
    x = make_inputs(2, nq, nk, d, seed=51, dtype=torch.float64)
    got, ref, _ = _run(x, d ** -0.5, causal, torch.bfloat16, "tcgen05")
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < TOL_BF16, n


def test_cotangent_scale_config():
    """Shape family of the causal D=128 configuration (cotangents ~ 0.1 N(0,1)), down-sized."""
    x = make_inputs(2, 512, 512, 128, seed=61, dtype=torch.float64, cot_scale=0.1)
    got, ref, _ = _run(x, 128 ** -0.5, True, torch.bfloat16, "tcgen05")
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < TOL_BF16, n


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
def test_reference_golden_fixture(impl):
    """The reference's own known-answer test (fhog/test_bwdbwd.py:27-82), all four outputs,
    with O recomputed by SDPA and L from produce_L exactly like that script does."""
    import fhob
    z = np.load(GOLDEN / "fhog_test_data.npz")
    t = {k: torch.from_numpy(z[k]).to(torch.bfloat16).cuda().unsqueeze(0) for k in z.files if z[k].ndim == 2}
    o = torch.nn.functional.scaled_dot_product_attention(t["q"], t["k"], t["v"], scale=0.125)
    L = fhob.produce_L(t["q"], t["k"], is_causal=False)
    got = fhob.flash_bwdbwd(t["q"], t["k"], t["v"], o, t["do"], t["ddq"], t["ddk"], t["ddv"], L, 0.125,
                            impl=impl, check=True)
    for n, g in zip(OUT_NAMES, got):
        assert O.rel_err(g[0], torch.from_numpy(z[n])) < TOL_BF16, n
    # element-wise check of the reference script (bf16 assert_close defaults), on the output it asserts
    torch.testing.assert_close(got[2][0].float().cpu(), torch.from_numpy(z["dv2"]), rtol=1.6e-2, atol=2e-2)


def test_reference_torch_vectors():
    """Outputs of the reference's torch restatement on seeded inputs (committed fixture)."""
    from golden.make_golden import TORCH_CASES, seeded_inputs
    import fhob
    z = np.load(GOLDEN / "ref_torch_closed_form.npz")
    for name, nq, nk, d, seed in TORCH_CASES:
        x = seeded_inputs(nq, nk, d, seed)
        scale = d ** -0.5
        lse = O.attn_lse(x["q"], x["k"], scale)
        o = O.attn_fwd(x["q"], x["k"], x["v"], scale)
        for dtype, tol in ((torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)):
            dev = {k: v.to(dtype).cuda().unsqueeze(0) for k, v in x.items()}
            got = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], o.to(dtype).cuda().unsqueeze(0), dev["do"],
                                    dev["ddq"], dev["ddk"], dev["ddv"], lse.float().cuda().unsqueeze(0), scale,
                                    check=True)
            for n, g in zip(OUT_NAMES, got):
                assert O.rel_err(g[0], torch.from_numpy(z[f"{name}/{n}"])) < tol, (name, n, dtype)


@pytest.mark.parametrize("causal", [False, True])
def test_forward_producer(causal):
    """attention_forward / produce_L against the oracle (O and fp32 LSE)."""
    import fhob
    x = make_inputs(2, 200, 328, 64, seed=71, dtype=torch.float64)
    o_ref = O.attn_fwd(x["q"], x["k"], x["v"], 0.125, causal)
    l_ref = O.attn_lse(x["q"], x["k"], 0.125, causal)
    o, lse = fhob.attention_forward(x["q"].float().cuda(), x["k"].float().cuda(), x["v"].float().cuda(), 0.125,
                                    is_causal=causal)
    assert O.rel_err(o, o_ref) < TOL_F32 and O.rel_err(lse, l_ref) < 1e-5
    o, lse = fhob.attention_forward(x["q"].bfloat16().cuda(), x["k"].bfloat16().cuda(), x["v"].bfloat16().cuda(),
                                    0.125, is_causal=causal)
    assert O.rel_err(o, o_ref) < TOL_BF16 and O.rel_err(lse, l_ref) < 1e-5


def _large_case(bh, nq, nk, d, causal, seed, cot_scale=1.0, heads_checked=(0,)):
    """Full-size run; the listed heads are checked against the chunked fp64 oracle on the GPU."""
    import fhob
    x = make_inputs(bh, nq, nk, d, seed=seed, dtype=torch.bfloat16, device="cuda", cot_scale=cot_scale,
                    on_device=bh * max(nq, nk) * d > 1 << 28)
    scale = d ** -0.5
    o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], scale, is_causal=causal)
    got = fhob.flash_bwdbwd(x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, scale,
                            is_causal=causal, check=True)
    for h in heads_checked:
        ref = O.bwdbwd_closed_form_chunked(*(x[n][h].double() for n in ("q", "k", "v", "do", "ddq", "ddk", "ddv")),
                                           scale, causal, chunk=1024)
        assert O.rel_err(lse[h], ref[4]) < 1e-5
        for n, g, r in zip(OUT_NAMES, got, ref[:4]):
            assert O.rel_err(g[h], r) < TOL_BF16, (n, h)
    return x, o, lse, got


def test_config_noncausal_2048_d64():
    _large_case(64, 2048, 2048, 64, False, seed=1234, heads_checked=(0, 63))


def test_config_causal_4096_d128():
    _large_case(128, 4096, 4096, 128, True, seed=1235, cot_scale=0.1, heads_checked=(0, 127))


def test_config_long_context_32768_d128():
    """The long-context causal configuration at full size (B=1, H=32, N=32768, D=128)."""
    _large_case(32, 32768, 32768, 128, True, seed=1236, heads_checked=(0, 31))


def test_config_cross_attention_4096x8192_d128():
    """A slice (8 heads) of the cross-attention scaling configuration; also the
    size-independent properties: bit-exact repeatability, head-shard invariance, linearity."""
    import fhob
    x, o, lse, got = _large_case(8, 4096, 8192, 128, False, seed=1237, heads_checked=(5,))
    scale = 128 ** -0.5
    args = lambda s, c=1.0: (x["q"][s], x["k"][s], x["v"][s], o[s], x["do"][s], x["ddq"][s] * c, x["ddk"][s] * c,
                             x["ddv"][s] * c, lse[s], scale)
    again = fhob.flash_bwdbwd(*args(slice(None)), check=True)
    for a, b in zip(got, again):
        assert torch.equal(a, b)                      # no atomics: bit-exact run to run
    shard = fhob.flash_bwdbwd(*args(slice(4, 8)), check=True)
    for a, b in zip(got, shard):
        assert torch.equal(a[4:8], b)                 # a head's result does not depend on its neighbours
    doubled = fhob.flash_bwdbwd(*args(slice(0, 2), 2.0), check=True)
    for a, b in zip(got, doubled):
        assert O.rel_err(b, 2.0 * a[0:2].float()) < 2e-2   # linear in the cotangents (powers of two: near exact)


def test_full_cross_attention_job_512_heads():
    """The whole cross-attention scaling job on one GPU (B=16, H=32 -> 512 heads, N_Q=4096, N_K=8192,
    D=128; 6.4 GB of inputs): first and last head against the fp64 oracle, and properties that hold
    bit for bit at any size - the operator is linear in (ddQ, ddK, ddV), doubling is exact in
    floating point, and a head's result does not depend on which launch it is part of."""
    import fhob
    x, o, lse, got = _large_case(512, 4096, 8192, 128, False, seed=1240, heads_checked=(0, 511))
    scale = 128 ** -0.5
    doubled = fhob.flash_bwdbwd(x["q"], x["k"], x["v"], o, x["do"], x["ddq"] * 2, x["ddk"] * 2, x["ddv"] * 2, lse,
                                scale, check=True)
    for n, a, b in zip(OUT_NAMES, got, doubled):
        assert torch.equal(b, a * 2), n
    del doubled
    for h in (0, 255, 511):
        s = slice(h, h + 1)
        alone = fhob.flash_bwdbwd(x["q"][s], x["k"][s], x["v"][s], o[s], x["do"][s], x["ddq"][s], x["ddk"][s],
                                  x["ddv"][s], lse[s], scale, check=True)
        for n, a, b in zip(OUT_NAMES, got, alone):
            assert torch.equal(a[s], b), (n, h)


@pytest.mark.parametrize("nq,nk", [(16384, 128), (128, 16384)])
def test_tensors_with_more_than_2_to_31_elements(nq, nk):
    """1025 heads x 16384 rows x 128 columns = 2.15e9 elements per tensor on one side: every offset
    beyond the first 2^31 elements (4 GiB) has to be computed in 64 bits.  The last head is the one
    that would show a wrapped offset."""
    x, o, lse, got = _large_case(1025, nq, nk, 128, False, seed=1241, heads_checked=(0, 1024))
    assert max(t.numel() for t in got) > 2 ** 31
    del x, o, lse, got
    torch.cuda.empty_cache()


@pytest.mark.parametrize("impl,dtype,tol", [("simt", torch.float32, TOL_F32), ("tcgen05", torch.bfloat16, TOL_BF16)])
def test_more_heads_than_one_grid_dimension_indexes(impl, dtype, tol):
    """70 000 heads of a tiny problem: the head index does not fit the y dimension of a launch grid."""
    import fhob
    bh = 70000
    x = make_inputs(bh, 40, 56, 16, seed=1242, dtype=dtype, device="cuda", on_device=True)
    o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], 0.25, is_causal=True, impl=impl)
    got = fhob.flash_bwdbwd(x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, 0.25,
                            is_causal=True, impl=impl, check=True)
    for h in (0, 65534, 65535, 65536, bh - 1):
        one = {n: t[h:h + 1].double().cpu() for n, t in x.items()}
        ref, lse_ref, _, _ = _oracle(one, 0.25, True)
        assert O.rel_err(lse[h:h + 1].cpu(), lse_ref) < 1e-4
        for n, g, r in zip(OUT_NAMES, got, ref):
            assert O.rel_err(g[h:h + 1].cpu(), r) < tol, (n, h)


def test_memory_is_linear_in_sequence_length():
    import fhob
    peaks = []
    for n in (2048, 4096, 8192):
        x = make_inputs(2, n, n, 64, seed=7, dtype=torch.bfloat16, device="cuda")
        o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], 0.125)
        torch.cuda.synchronize()
        fhob.ops._workspaces.clear()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        fhob.flash_bwdbwd(x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, 0.125, check=True)
        peaks.append(torch.cuda.max_memory_allocated() - base)
    io_bytes = [4 * 2 * n * 64 * 2 for n in (2048, 4096, 8192)]      # the four outputs
    for pk, io in zip(peaks, io_bytes):
        assert pk <= io + (1 << 20) + 2 * (1 << 20)   # outputs + workspace floor (1 MiB) + allocator rounding
    assert peaks[2] < 4.5 * max(peaks[0], 1 << 20)    # 4x the length -> ~4x, not 16x


def test_host_buffers_end_to_end():
    """The host-buffer form of the entry point (pinned host tensors in, host tensors out)."""
    import fhob
    x = make_inputs(2, 256, 256, 64, seed=81, dtype=torch.float64)
    ref, lse, o, _ = _oracle(x, 0.125, False)
    host = {k: v.bfloat16().pin_memory() for k, v in x.items()}
    got = fhob.flash_bwdbwd(host["q"], host["k"], host["v"], o.bfloat16().pin_memory(), host["do"], host["ddq"],
                            host["ddk"], host["ddv"], lse.float().pin_memory(), 0.125, check=True)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert g.device.type == "cpu"
        assert O.rel_err(g, r) < TOL_BF16, n
    # many ranges (one head each), more than the ring of staging sets holds, into caller-owned tensors, twice
    x = make_inputs(9, 192, 320, 64, seed=82, dtype=torch.float64)
    ref, lse, o, _ = _oracle(x, 0.125, True)
    host = {k: v.bfloat16().pin_memory() for k, v in x.items()}
    outs = tuple(torch.empty(t.shape, dtype=torch.bfloat16).pin_memory() for t in (x["q"], x["k"], x["k"], x["q"]))
    saved = fhob.ops.HOST_RANGE_BYTES
    try:
        fhob.ops.HOST_RANGE_BYTES = 1      # one head per range
        for _ in range(2):
            for t in outs:
                t.zero_()
            got = fhob.flash_bwdbwd(host["q"], host["k"], host["v"], o.bfloat16().pin_memory(), host["do"],
                                    host["ddq"], host["ddk"], host["ddv"], lse.float().pin_memory(), 0.125,
                                    is_causal=True, out=outs)
            for n, g, t, r in zip(OUT_NAMES, got, outs, ref):
                assert g.data_ptr() == t.data_ptr()
                assert O.rel_err(g, r) < TOL_BF16, n
        # without the saved forward output: it is not uploaded at all
        got = fhob.flash_bwdbwd(host["q"], host["k"], host["v"], None, host["do"], host["ddq"], host["ddk"],
                                host["ddv"], lse.float().pin_memory(), 0.125, is_causal=True)
        for n, g, r in zip(OUT_NAMES, got, ref):
            assert O.rel_err(g, r) < TOL_BF16, n
    finally:
        fhob.ops.HOST_RANGE_BYTES = saved
    # the staging sets and workspaces the module keeps between calls can be given back
    del got
    before = torch.cuda.memory_allocated()
    fhob.release_cached_memory()
    assert torch.cuda.memory_allocated() < before and not fhob.ops._staging and not fhob.ops._workspaces


def test_empty_problems_on_the_device():
    """No keys: O = 0, L = -inf, every gradient zero; an empty batch: empty results.  Nothing is launched."""
    import fhob
    q = torch.randn(2, 16, 64, device="cuda", dtype=torch.bfloat16)
    k, v = q[:, :0], q[:, :0, :32]
    o, lse = fhob.attention_forward(q, k, v, 0.125)
    assert o.shape == (2, 16, 32) and not o.any() and torch.isneginf(lse).all()
    assert torch.isneginf(fhob.produce_L(q, k)).all()
    got = fhob.flash_bwdbwd(q, k, v, o, o, q, k, v, lse, 0.125, check=True)
    assert [tuple(t.shape) for t in got] == [(2, 16, 64), (2, 0, 64), (2, 0, 32), (2, 16, 32)]
    assert not got[0].any() and not got[3].any()
    e = q[:0]
    assert fhob.attention_forward(e, e, e)[0].shape == (0, 16, 64)
    assert all(t.numel() == 0 for t in fhob.flash_bwdbwd(e, e, e, e, e, e, e, e, e[:, :, 0].float(), 0.125))


def test_wrong_inputs_raise():
    import fhob
    q = torch.zeros(2, 128, 64, device="cuda", dtype=torch.bfloat16)
    L = torch.zeros(2, 128, device="cuda")
    with pytest.raises(TypeError):
        fhob.flash_bwdbwd(q, q, q, q, q.float(), q, q, q, L, 0.125)
    with pytest.raises(ValueError):
        fhob.flash_bwdbwd(q, q[:, :64], q, q, q, q, q, q, L, 0.125)
    with pytest.raises(ValueError):
        fhob.flash_bwdbwd(q, q, q, q, q, q, q, q, L[:, :64], 0.125)
    with pytest.raises(TypeError):
        qd = q.double()
        fhob.flash_bwdbwd(qd, qd, qd, qd, qd, qd, qd, qd, L, 0.125)
    q36 = torch.zeros(2, 128, 36, device="cuda", dtype=torch.bfloat16)    # rows of 72 bytes: not 16-byte aligned
    with pytest.raises(RuntimeError, match="shape not supported"):
        fhob.flash_bwdbwd(q36, q36, q36, q36, q36, q36, q36, q36, L, 0.125, impl="tcgen05")


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)])
def test_first_backward(dtype, tol, causal):
    """fhob_backward against the oracle's attn_bwd (jax_refs/flash_impl.py:124-173)."""
    import fhob
    x = make_inputs(2, 200, 328, 64, seed=91, dtype=torch.float64)
    ref = O.attn_bwd(x["q"], x["k"], x["v"], x["do"], 0.125, causal)
    o = O.attn_fwd(x["q"], x["k"], x["v"], 0.125, causal)
    lse = O.attn_lse(x["q"], x["k"], 0.125, causal)
    dev = {k: v.to(dtype).cuda() for k, v in x.items()}
    got = fhob.attention_backward(dev["q"], dev["k"], dev["v"], o.to(dtype).cuda(), dev["do"], lse.float().cuda(),
                                  0.125, is_causal=causal)
    for n, g, r in zip(("dq", "dk", "dv"), got, ref):
        assert O.rel_err(g, r) < tol, n


@pytest.mark.parametrize("causal", [False, True])
def test_autograd_grad_of_grad(causal):
    """torch.autograd.grad twice through fhob.attention equals the oracle's grad-of-grad (form A):
    the use the reference's commented-out Bwd function was meant for (fhog/triton_bwdbwd.py:538-554)."""
    import fhob
    x = make_inputs(2, 128, 256, 64, seed=93, dtype=torch.float64)
    ref = O.bwdbwd_autograd(*x.values(), 0.125, causal)
    ref_first = O.attn_bwd(x["q"], x["k"], x["v"], x["do"], 0.125, causal)
    for dtype, tol in ((torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)):
        q, k, v, do = (x[n].to(dtype).cuda().requires_grad_(True) for n in ("q", "k", "v", "do"))
        out = fhob.attention(q, k, v, 0.125, is_causal=causal)
        dq, dk, dv = torch.autograd.grad(out, (q, k, v), do, create_graph=True)
        for n, g, r in zip(("dq", "dk", "dv"), (dq, dk, dv), ref_first):
            assert O.rel_err(g.detach(), r) < tol, (n, dtype)
        cot = tuple(x[n].to(dtype).cuda() for n in ("ddq", "ddk", "ddv"))
        got = torch.autograd.grad((dq, dk, dv), (q, k, v, do), cot)
        for n, g, r in zip(OUT_NAMES, got, ref):
            assert O.rel_err(g, r) < tol, (n, dtype)


# ---- sliding window (sliding_window_length of jax_refs/flash_impl.py:86-91)

WINDOW_CASES = [
    # bh, nq, nk, d, window
    (2, 256, 256, 64, 17),     # narrower than a tile
    (2, 384, 384, 128, 64),    # exactly one streamed tile
    (1, 512, 512, 128, 200),   # spans several tiles, not a multiple of any tile size
    (2, 256, 448, 64, 100),    # more keys than queries: leading keys are visible to no query
    (1, 200, 328, 128, 77),    # ragged lengths
    (1, 256, 256, 64, 4096),   # window wider than the sequence = plain causal
]


def _window_case(bh, nq, nk, d, w, dtype, impl):
    import fhob
    x = make_inputs(bh, nq, nk, d, seed=101, dtype=torch.float64)
    scale = d ** -0.5
    ref = O.bwdbwd_closed_form(*x.values(), scale, True, sliding_window_length=w)
    o = O.attn_fwd(x["q"], x["k"], x["v"], scale, True, sliding_window_length=w)
    lse = O.attn_lse(x["q"], x["k"], scale, True, sliding_window_length=w)
    dev = {k: v.to(dtype).cuda() for k, v in x.items()}
    got = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], o.to(dtype).cuda(), dev["do"], dev["ddq"], dev["ddk"],
                            dev["ddv"], lse.float().cuda(), scale, is_causal=True, sliding_window=w, impl=impl,
                            check=True)
    return got, ref


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("bh,nq,nk,d,w", WINDOW_CASES)
def test_bf16_sliding_window(bh, nq, nk, d, w, impl):
    got, ref = _window_case(bh, nq, nk, d, w, torch.bfloat16, impl)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < TOL_BF16, n


@pytest.mark.parametrize("bh,nq,nk,d,w", WINDOW_CASES[:4])
def test_fp32_sliding_window(bh, nq, nk, d, w):
    got, ref = _window_case(bh, nq, nk, d, w, torch.float32, "auto")
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < TOL_F32, n


def test_sliding_window_keys_outside_every_window_get_zero():
    """With more keys than queries the first keys lie before every query's window."""
    got, _ = _window_case(1, 128, 512, 64, 32, torch.bfloat16, "tcgen05")
    n_dead = 512 - 128 - 32 + 1   # keys j with (0 + n_k - n_q) - j >= window
    assert torch.count_nonzero(got[1][:, :n_dead]) == 0 and torch.count_nonzero(got[2][:, :n_dead]) == 0
    assert torch.count_nonzero(got[1][:, n_dead]) > 0


def test_sliding_window_forward_backward_and_autograd():
    """Forward producer, first backward and the twice-differentiable function with a window."""
    import fhob
    w, scale = 50, 0.125
    x = make_inputs(2, 192, 256, 64, seed=103, dtype=torch.float64)
    o_ref = O.attn_fwd(x["q"], x["k"], x["v"], scale, True, sliding_window_length=w)
    lse_ref = O.attn_lse(x["q"], x["k"], scale, True, sliding_window_length=w)
    first_ref = O.attn_bwd(x["q"], x["k"], x["v"], x["do"], scale, True, sliding_window_length=w)
    ref = O.bwdbwd_autograd(*x.values(), scale, True, sliding_window_length=w)
    q, k, v, do = (x[n].float().cuda().requires_grad_(True) for n in ("q", "k", "v", "do"))
    o, lse = fhob.attention_forward(q.detach(), k.detach(), v.detach(), scale, is_causal=True, sliding_window=w)
    assert O.rel_err(o, o_ref) < TOL_F32 and O.rel_err(lse, lse_ref) < TOL_F32
    out = fhob.attention(q, k, v, scale, is_causal=True, sliding_window=w)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do, create_graph=True)
    for n, g, r in zip(("dq", "dk", "dv"), (dq, dk, dv), first_ref):
        assert O.rel_err(g.detach(), r) < TOL_F32, n
    cot = tuple(x[n].float().cuda() for n in ("ddq", "ddk", "ddv"))
    got = torch.autograd.grad((dq, dk, dv), (q, k, v, do), cot)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < TOL_F32, n


def test_sliding_window_argument_errors():
    import fhob
    x = {k: v.bfloat16().cuda() for k, v in make_inputs(1, 128, 128, 64, seed=105, dtype=torch.float32).items()}
    o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], 0.125)
    args = (x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, 0.125)
    with pytest.raises(ValueError):
        fhob.flash_bwdbwd(*args, sliding_window=16)              # needs is_causal
    with pytest.raises(ValueError):
        fhob.flash_bwdbwd(*args, is_causal=True, sliding_window=0)
    with pytest.raises(ValueError):
        fhob.flash_bwdbwd(*args, is_causal=True, sliding_window=2.5)


# ---- float16 storage (the dtype of the reference's benchmark script, fhog/benchhhh.py:19)

@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("bh,nq,nk,d", [(2, 256, 384, 64), (2, 384, 384, 128), (1, 200, 328, 128)])
def test_fp16_outputs(bh, nq, nk, d, causal, impl):
    x = make_inputs(bh, nq, nk, d, seed=111, dtype=torch.float64)
    # the oracle sees the fp16-rounded inputs, like the operator
    x = {k: v.half().double() for k, v in x.items()}
    got, ref, _ = _run(x, d ** -0.5, causal, torch.float16, impl)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert g.dtype == torch.float16
        assert O.rel_err(g, r) < 5e-3, n      # 11-bit significand: tighter than the bf16 bound


def test_fp16_forward_backward_autograd():
    import fhob
    x = make_inputs(2, 128, 256, 64, seed=113, dtype=torch.float64)
    x = {k: v.half().double() for k, v in x.items()}
    ref = O.bwdbwd_autograd(*x.values(), 0.125, True)
    q, k, v, do = (x[n].half().cuda().requires_grad_(True) for n in ("q", "k", "v", "do"))
    out = fhob.attention(q, k, v, 0.125, is_causal=True)
    assert out.dtype == torch.float16
    assert O.rel_err(out.detach(), O.attn_fwd(x["q"], x["k"], x["v"], 0.125, True)) < 2e-3
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do, create_graph=True)
    cot = tuple(x[n].half().cuda() for n in ("ddq", "ddk", "ddv"))
    got = torch.autograd.grad((dq, dk, dv), (q, k, v, do), cot)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < 1e-2, n


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_reproduce_one_gpu_bit_for_bit():
    """Head shards on two devices driven from one process give exactly the rows one device gives:
    no collective, no peer access, and each call runs on the device of its tensors."""
    import fhob
    from fhob.sharding import sharded_call
    x = make_inputs(6, 256, 384, 128, seed=121, dtype=torch.bfloat16, device="cuda:0")
    scale = 128 ** -0.5
    o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], scale, is_causal=True)
    names = ("q", "k", "v", "o", "do", "ddq", "ddk", "ddv", "lse")
    full = dict(x, o=o, lse=lse)
    ref = fhob.flash_bwdbwd(*(full[n] for n in names), scale, is_causal=True, check=True)
    for rank in range(2):
        dev = torch.device("cuda", rank)
        moved = [full[n].to(dev) for n in names]
        start, count, got = sharded_call(
            lambda *t: fhob.flash_bwdbwd(*t, scale, is_causal=True, check=True), moved, 6, 2, rank)
        assert count == 3
        for g, r in zip(got, ref):
            assert g.device == dev
            assert torch.equal(g.cpu(), r[start:start + count].cpu())


# ---- forward and first backward on both kernel families

FO_CASES = [(2, 256, 384, 64), (2, 384, 384, 128), (1, 200, 328, 128), (3, 128, 512, 64), (1, 640, 640, 128)]


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
@pytest.mark.parametrize("causal,window", [(False, None), (True, None), (True, 70)])
@pytest.mark.parametrize("bh,nq,nk,d", FO_CASES)
def test_bf16_forward_and_first_backward(bh, nq, nk, d, causal, window, impl):
    import fhob
    import math
    w = math.inf if window is None else window
    x = make_inputs(bh, nq, nk, d, seed=131, dtype=torch.float64)
    scale = d ** -0.5
    o_ref = O.attn_fwd(x["q"], x["k"], x["v"], scale, causal, sliding_window_length=w)
    l_ref = O.attn_lse(x["q"], x["k"], scale, causal, sliding_window_length=w)
    first_ref = O.attn_bwd(x["q"], x["k"], x["v"], x["do"], scale, causal, sliding_window_length=w)
    dev = {k: v.bfloat16().cuda() for k, v in x.items()}
    o, lse = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, is_causal=causal, sliding_window=window,
                                    impl=impl)
    assert o.dtype == torch.bfloat16 and lse.dtype == torch.float32
    assert O.rel_err(o, o_ref) < TOL_BF16 and O.rel_err(lse, l_ref) < 1e-5
    got = fhob.attention_backward(dev["q"], dev["k"], dev["v"], o_ref.bfloat16().cuda(), dev["do"],
                                  l_ref.float().cuda(), scale, is_causal=causal, sliding_window=window, impl=impl)
    for n, g, r in zip(("dq", "dk", "dv"), got, first_ref):
        assert O.rel_err(g, r) < TOL_BF16, n


def test_tensor_core_forward_is_reproducible_and_matches_cuda_cores():
    import fhob
    x = make_inputs(4, 512, 768, 128, seed=133, dtype=torch.bfloat16, device="cuda")
    a = fhob.attention_forward(x["q"], x["k"], x["v"], 0.09, is_causal=True, impl="tcgen05")
    b = fhob.attention_forward(x["q"], x["k"], x["v"], 0.09, is_causal=True, impl="tcgen05")
    c = fhob.attention_forward(x["q"], x["k"], x["v"], 0.09, is_causal=True, impl="simt")
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert O.rel_err(a[0], c[0].double()) < 1e-2 and O.rel_err(a[1], c[1].double()) < 1e-5


# ---- seeded random shapes: tile-range and masking logic of every tensor-core kernel

def _random_cases(n, seed):
    import random
    rng = random.Random(seed)
    cases = []
    while len(cases) < n:
        d = rng.choice([64, 128])
        nq = rng.randint(1, 440)                 # any length: the row vectors are padded per head
        nk = rng.randint(1, 450)
        causal = rng.random() < 0.6
        if causal and nk < nq:
            nk = nq + rng.randint(0, 64)         # every query keeps at least one visible key
        window = rng.choice([None, None, rng.randint(1, 300)]) if causal else None
        cases.append((rng.randint(1, 3), nq, nk, d, causal, window))
    return cases


@pytest.mark.parametrize("bh,nq,nk,d,causal,window", _random_cases(24, seed=2024))
def test_random_shapes_all_tensor_core_kernels(bh, nq, nk, d, causal, window):
    import fhob
    import math
    w = math.inf if window is None else window
    x = make_inputs(bh, nq, nk, d, seed=nq * 1000 + nk, dtype=torch.float64)
    scale = d ** -0.5
    o_ref = O.attn_fwd(x["q"], x["k"], x["v"], scale, causal, sliding_window_length=w)
    l_ref = O.attn_lse(x["q"], x["k"], scale, causal, sliding_window_length=w)
    first_ref = O.attn_bwd(x["q"], x["k"], x["v"], x["do"], scale, causal, sliding_window_length=w)
    ref = O.bwdbwd_closed_form(*x.values(), scale, causal, sliding_window_length=w)
    dev = {k: v.bfloat16().cuda() for k, v in x.items()}
    kw = dict(is_causal=causal, sliding_window=window, impl="tcgen05")
    o, lse = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, **kw)
    assert O.rel_err(o, o_ref) < TOL_BF16 and O.rel_err(lse, l_ref) < 1e-5
    first = fhob.attention_backward(dev["q"], dev["k"], dev["v"], o, dev["do"], lse, scale, **kw)
    for n, g, r in zip(("dq", "dk", "dv"), first, first_ref):
        assert O.rel_err(g, r) < TOL_BF16, n
    got = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], o, dev["do"], dev["ddq"], dev["ddk"], dev["ddv"], lse,
                            scale, check=True, **kw)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < TOL_BF16, n


def _random_mixed_cases(n, seed):
    """Random head dims (two of them), storage types, masks and lengths, including causal problems
    with fewer keys than queries; fp32 cases keep both head dims at most 64 (the tensor-core path)."""
    import random
    rng = random.Random(seed)
    cases = []
    while len(cases) < n:
        dtype = rng.choice(["bf16", "bf16", "f16", "f32"])
        top = 8 if dtype == "f32" else 16
        d, dv = 8 * rng.randint(1, top), 8 * rng.randint(1, top)
        nq, nk = rng.randint(1, 330), rng.randint(1, 330)
        causal = rng.random() < 0.5
        window = rng.choice([None, rng.randint(1, 200)]) if causal else None
        cases.append((rng.randint(1, 3), nq, nk, d, dv, dtype, causal, window))
    return cases


@pytest.mark.parametrize("bh,nq,nk,d,dv,dtype,causal,window", _random_mixed_cases(48, seed=2025))
def test_random_head_dims_types_and_masks_on_the_tensor_cores(bh, nq, nk, d, dv, dtype, causal, window):
    """The tensor-core kernels (operator, forward, first backward) on random problems."""
    import fhob
    import math
    tdt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    tol = TOL_F32 if dtype == "f32" else TOL_BF16
    g = torch.Generator().manual_seed(nq * 1000 + nk + d)
    mk = lambda n, dd: torch.randn(bh, n, dd, generator=g, dtype=torch.float64).to(tdt).double()
    x = dict(q=mk(nq, d), k=mk(nk, d), v=mk(nk, dv), do=mk(nq, dv), ddq=mk(nq, d), ddk=mk(nk, d), ddv=mk(nk, dv))
    scale = d ** -0.5
    w = math.inf if window is None else window
    dead = nq - nk if (causal and nk < nq) else 0   # queries without any visible key: oracle on the rest
    live = {n: (t[:, dead:] if n in ("q", "do", "ddq") else t) for n, t in x.items()}
    r = O.bwdbwd_closed_form(*live.values(), scale, causal, sliding_window_length=w)
    first = O.attn_bwd(live["q"], live["k"], live["v"], live["do"], scale, causal, sliding_window_length=w)
    o_live = O.attn_fwd(live["q"], live["k"], live["v"], scale, causal, sliding_window_length=w)
    l_live = O.attn_lse(live["q"], live["k"], scale, causal, sliding_window_length=w)
    zq, zv = torch.zeros_like(x["q"][:, :dead]), torch.zeros_like(x["do"][:, :dead])
    ref = (torch.cat([zq, r[0]], 1), r[1], r[2], torch.cat([zv, r[3]], 1))
    first_ref = (torch.cat([zq, first[0]], 1), first[1], first[2])
    dev = {n: t.to(tdt).cuda() for n, t in x.items()}
    kw = dict(is_causal=causal, sliding_window=window, impl="tcgen05")
    o, lse = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, **kw)
    assert O.rel_err(o[:, dead:], o_live) < tol and O.rel_err(lse[:, dead:], l_live) < 1e-4
    assert not o[:, :dead].any() and torch.isneginf(lse[:, :dead]).all()
    got_first = fhob.attention_backward(dev["q"], dev["k"], dev["v"], o, dev["do"], lse, scale, **kw)
    got = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], o, dev["do"], dev["ddq"], dev["ddk"], dev["ddv"], lse,
                            scale, check=True, **kw)
    for n, a, rr in list(zip(("dq", "dk", "dv"), got_first, first_ref)) + list(zip(OUT_NAMES, got, ref)):
        assert torch.isfinite(a).all(), n
        # against the tensor's abs-max, or against 1e-3 where the exact result vanishes (a query row
        # with a single visible key has no second-order terms: the kernels then return rounding noise)
        err = float((a.double().cpu() - rr).abs().max() / max(float(rr.abs().max()), 1e-3)) if rr.numel() else 0.0
        assert err < tol, (n, err)


def _random_simt_cases(n, seed):
    import random
    rng = random.Random(seed)
    cases = []
    while len(cases) < n:
        dtype = rng.choice(["f32", "f32", "bf16"])
        step = 4 if dtype == "f32" else 8           # rows stay 16-byte aligned
        d, dv = step * rng.randint(1, 128 // step), step * rng.randint(1, 128 // step)
        nq, nk = rng.randint(1, 200), rng.randint(1, 200)
        causal = rng.random() < 0.5
        window = rng.choice([None, rng.randint(1, 150)]) if causal else None
        cases.append((rng.randint(1, 3), nq, nk, d, dv, dtype, causal, window))
    return cases


@pytest.mark.parametrize("bh,nq,nk,d,dv,dtype,causal,window", _random_simt_cases(24, seed=2026))
def test_random_head_dims_types_and_masks_on_the_cuda_cores(bh, nq, nk, d, dv, dtype, causal, window):
    """The CUDA-core kernels (operator, forward, first backward) on random problems: any head dims up
    to 128 that keep rows 16-byte aligned, two of them, both storage classes, every mask."""
    import fhob
    import math
    tdt = {"bf16": torch.bfloat16, "f32": torch.float32}[dtype]
    tol = TOL_F32 if dtype == "f32" else TOL_BF16
    g = torch.Generator().manual_seed(nq * 1000 + nk + d)
    mk = lambda n, dd: torch.randn(bh, n, dd, generator=g, dtype=torch.float64).to(tdt).double()
    x = dict(q=mk(nq, d), k=mk(nk, d), v=mk(nk, dv), do=mk(nq, dv), ddq=mk(nq, d), ddk=mk(nk, d), ddv=mk(nk, dv))
    scale = d ** -0.5
    w = math.inf if window is None else window
    dead = nq - nk if (causal and nk < nq) else 0   # queries without any visible key: oracle on the rest
    live = {n: (t[:, dead:] if n in ("q", "do", "ddq") else t) for n, t in x.items()}
    r = O.bwdbwd_closed_form(*live.values(), scale, causal, sliding_window_length=w)
    first = O.attn_bwd(live["q"], live["k"], live["v"], live["do"], scale, causal, sliding_window_length=w)
    zq, zv = torch.zeros_like(x["q"][:, :dead]), torch.zeros_like(x["do"][:, :dead])
    ref = (torch.cat([zq, r[0]], 1), r[1], r[2], torch.cat([zv, r[3]], 1))
    first_ref = (torch.cat([zq, first[0]], 1), first[1], first[2])
    dev = {n: t.to(tdt).cuda() for n, t in x.items()}
    kw = dict(is_causal=causal, sliding_window=window, impl="simt")
    o, lse = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, **kw)
    got_first = fhob.attention_backward(dev["q"], dev["k"], dev["v"], o, dev["do"], lse, scale, **kw)
    got = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], o, dev["do"], dev["ddq"], dev["ddk"], dev["ddv"], lse,
                            scale, check=True, **kw)
    for n, a, rr in list(zip(("dq", "dk", "dv"), got_first, first_ref)) + list(zip(OUT_NAMES, got, ref)):
        assert torch.isfinite(a).all(), n
        err = float((a.double().cpu() - rr).abs().max() / max(float(rr.abs().max()), 1e-3)) if rr.numel() else 0.0
        assert err < tol, (n, err)


def test_expired_wait_is_reported_and_leaves_the_context_usable():
    """A device wait that can never complete gives up after about a second, sets FHOB_ERR_TIMEOUT
    in the status word and the kernel returns; the next operator call clears the word and works."""
    import ctypes as C
    import fhob
    from fhob import _lib
    lib = _lib.load()
    x = make_inputs(1, 128, 128, 64, seed=141, dtype=torch.bfloat16, device="cuda")
    ws = torch.zeros(lib.fhob_workspace_bytes(1, 128), dtype=torch.uint8, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.fhob_selftest_expired_wait(C.c_void_p(ws.data_ptr()), ws.numel(), stream) == 0
    p = _lib.FhobProblem()
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    assert lib.fhob_read_status(C.byref(p), stream) == _lib.ERR_TIMEOUT
    with pytest.raises(RuntimeError, match="status 64"):
        _lib.check(_lib.ERR_TIMEOUT, "self-test")
    o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], 0.125)
    got = fhob.flash_bwdbwd(x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, 0.125,
                            check=True)
    assert all(torch.isfinite(g.float()).all() for g in got)


def test_cuda_graph_capture_and_replay():
    """The operator only queues kernels on the current stream (no synchronisation, no allocation
    of its own on the success path), so a call can be captured into a CUDA graph and replayed on
    new input values; replays reproduce the eager results bit for bit."""
    import fhob
    scale = 0.125
    static = make_inputs(4, 256, 384, 64, seed=151, dtype=torch.bfloat16, device="cuda")
    o, lse = fhob.attention_forward(static["q"], static["k"], static["v"], scale, is_causal=True)
    args = lambda: (static["q"], static["k"], static["v"], o, static["do"], static["ddq"], static["ddk"],
                    static["ddv"], lse, scale)
    fhob.flash_bwdbwd(*args(), is_causal=True)          # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o_g, lse_g = fhob.attention_forward(static["q"], static["k"], static["v"], scale, is_causal=True)
        outs = fhob.flash_bwdbwd(static["q"], static["k"], static["v"], o_g, static["do"], static["ddq"],
                                 static["ddk"], static["ddv"], lse_g, scale, is_causal=True)
    for seed in (152, 153):
        fresh = make_inputs(4, 256, 384, 64, seed=seed, dtype=torch.bfloat16, device="cuda")
        for k in static:
            static[k].copy_(fresh[k])
        graph.replay()
        torch.cuda.synchronize()
        o_e, lse_e = fhob.attention_forward(fresh["q"], fresh["k"], fresh["v"], scale, is_causal=True)
        eager = fhob.flash_bwdbwd(fresh["q"], fresh["k"], fresh["v"], o_e, fresh["do"], fresh["ddq"], fresh["ddk"],
                                  fresh["ddv"], lse_e, scale, is_causal=True, check=True)
        assert torch.equal(o_g, o_e) and torch.equal(lse_g, lse_e)
        for g, e in zip(outs, eager):
            assert torch.equal(g, e)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
def test_bf16_without_saved_output(d, causal):
    """O=None: D = rowsum(dO * O) is replaced by sum_j P dP, accumulated by the sweep that yields dd
    and b.  Same results within the bf16 bound, and close to the call that passes O."""
    import fhob
    x = make_inputs(2, 384, 512, d, seed=161, dtype=torch.float64)
    scale = d ** -0.5
    ref = O.bwdbwd_closed_form(*x.values(), scale, causal)
    lse = O.attn_lse(x["q"], x["k"], scale, causal).float().cuda()
    o = O.attn_fwd(x["q"], x["k"], x["v"], scale, causal).bfloat16().cuda()
    dev = {k: v.bfloat16().cuda() for k, v in x.items()}
    rest = (dev["do"], dev["ddq"], dev["ddk"], dev["ddv"], lse, scale)
    got = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], None, *rest, is_causal=causal, check=True)
    with_o = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], o, *rest, is_causal=causal, check=True)
    for n, g, w, r in zip(OUT_NAMES, got, with_o, ref):
        assert O.rel_err(g, r) < TOL_BF16, n
        assert O.rel_err(g, w.double()) < 1e-2, n
    stats = fhob.run_passes(dev["q"], dev["k"], dev["v"], None, *rest, is_causal=causal, upto=2, fused12=True)
    sd, sdd, sb = O.bwdbwd_row_stats(*x.values(), scale, causal)
    assert O.rel_err(stats["d"], sd) < 5e-3 and O.rel_err(stats["dd"], sdd) < TOL_BF16
    assert O.rel_err(stats["b"], sb) < TOL_BF16
    with pytest.raises(RuntimeError, match="invalid argument"):
        fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], None, *rest, is_causal=causal, impl="simt")


@pytest.mark.parametrize("impl", ["simt", "tcgen05"])
def test_logsumexp_only_forward(impl):
    """produce_L / need_o=False: the scores reduced to the fp32 logsumexp, no P V product
    (role of produce_L, fhog/triton_flash.py:252-258, which is dense, bf16 and non-causal only)."""
    import fhob
    import math
    for (bh, nq, nk, d, causal, w) in [(2, 384, 640, 128, False, None), (2, 328, 328, 64, True, None),
                                       (1, 512, 700, 128, True, 150)]:
        x = make_inputs(bh, nq, nk, d, seed=171, dtype=torch.float64)
        scale = d ** -0.5
        l_ref = O.attn_lse(x["q"], x["k"], scale, causal, sliding_window_length=math.inf if w is None else w)
        q, k = x["q"].bfloat16().cuda(), x["k"].bfloat16().cuda()
        o, lse = fhob.attention_forward(q, k, k, scale, is_causal=causal, sliding_window=w, impl=impl, need_o=False,
                                        check=True)
        assert o is None and lse.dtype == torch.float32
        assert O.rel_err(lse, l_ref) < 1e-5, (bh, nq, nk, d, causal, w)
    assert O.rel_err(fhob.produce_L(q, k, is_causal=True, scale=scale, sliding_window=150), l_ref) < 1e-5


def _live_rows_oracle(x, scale, first_live, window=None):
    """Oracle results of a causal problem with n_k < n_q: the first `first_live` queries see no
    key, so the problem equals the one over the remaining queries (the mask is bottom-right
    aligned), with zero rows for the dead queries in the query-shaped results."""
    import math
    w = math.inf if window is None else window
    live = {n: (t[:, first_live:] if n in ("q", "do", "ddq") else t) for n, t in x.items()}
    ref = O.bwdbwd_closed_form(*live.values(), scale, True, sliding_window_length=w)
    pad = lambda t: torch.cat([torch.zeros_like(x["q"][:, :first_live]), t], dim=1)
    return (pad(ref[0]), ref[1], ref[2], pad(ref[3])), live


@pytest.mark.parametrize("dtype,impl,tol", [(torch.bfloat16, "tcgen05", TOL_BF16), (torch.bfloat16, "simt", TOL_BF16),
                                            (torch.float32, "auto", TOL_F32)])
@pytest.mark.parametrize("bh,nq,nk,d,window", [(2, 384, 256, 128, None), (1, 300, 90, 64, None), (2, 256, 128, 64, 40),
                                               (1, 517, 130, 128, None)])
def test_causal_queries_without_any_visible_key(bh, nq, nk, d, window, dtype, impl, tol):
    """Causal with n_k < n_q: the first n_q - n_k queries see no key.  Their dQ2 and ddO rows are
    exactly zero, they add nothing to dK2 and dV2, and whatever sits in their rows of O and L
    (NaN and -inf here, what a softmax over an empty row gives) is not read.  The reference
    leaves the case undefined (its operator has no causal mask, its oracle divides 0 by 0)."""
    import fhob
    first_live = nq - nk
    x = make_inputs(bh, nq, nk, d, seed=311, dtype=torch.float64)
    scale = d ** -0.5
    ref, live = _live_rows_oracle(x, scale, first_live, window)
    import math
    wl = math.inf if window is None else window
    o_live = O.attn_fwd(live["q"], live["k"], live["v"], scale, True, sliding_window_length=wl)
    l_live = O.attn_lse(live["q"], live["k"], scale, True, sliding_window_length=wl)
    o = torch.cat([torch.full_like(x["q"][:, :first_live], float("nan")), o_live], dim=1)
    lse = torch.cat([torch.full((bh, first_live), -float("inf"), dtype=torch.float64), l_live], dim=1)
    dev = {k: v.to(dtype).cuda() for k, v in x.items()}
    kw = dict(is_causal=True, sliding_window=window, impl=impl)
    got = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], o.to(dtype).cuda(), dev["do"], dev["ddq"], dev["ddk"],
                            dev["ddv"], lse.float().cuda(), scale, check=True, **kw)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert torch.isfinite(g).all(), n
        assert O.rel_err(g, r) < tol, n
    assert torch.count_nonzero(got[0][:, :first_live]) == 0 and torch.count_nonzero(got[3][:, :first_live]) == 0
    # the library's own forward gives O = 0 and L = -inf on those rows, and the first backward zero dQ rows
    o_dev, lse_dev = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, **kw)
    assert torch.count_nonzero(o_dev[:, :first_live]) == 0 and torch.isinf(lse_dev[:, :first_live]).all()
    assert O.rel_err(o_dev[:, first_live:], o_live) < tol
    first = fhob.attention_backward(dev["q"], dev["k"], dev["v"], o_dev, dev["do"], lse_dev, scale, **kw)
    first_ref = O.attn_bwd(live["q"], live["k"], live["v"], live["do"], scale, True, sliding_window_length=wl)
    assert torch.count_nonzero(first[0][:, :first_live]) == 0
    assert O.rel_err(first[0][:, first_live:], first_ref[0]) < tol
    assert O.rel_err(first[1], first_ref[1]) < tol and O.rel_err(first[2], first_ref[2]) < tol
    if dtype != torch.float32 and impl == "tcgen05":
        # without the saved output (D from the sweep) the same holds
        got2 = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], None, dev["do"], dev["ddq"], dev["ddk"], dev["ddv"],
                                 lse.float().cuda(), scale, check=True, **kw)
        for n, g, r in zip(OUT_NAMES, got2, ref):
            assert torch.isfinite(g).all() and O.rel_err(g, r) < tol, n


def _two_dim_inputs(bh, nq, nk, dqk, dv, seed):
    g = torch.Generator().manual_seed(seed)
    shapes = dict(q=(bh, nq, dqk), k=(bh, nk, dqk), v=(bh, nk, dv), do=(bh, nq, dv),
                  ddq=(bh, nq, dqk), ddk=(bh, nk, dqk), ddv=(bh, nk, dv))
    return {n: torch.randn(s, generator=g).bfloat16().double() for n, s in shapes.items()}


@pytest.mark.parametrize("dtype,impl,tol", [(torch.bfloat16, "tcgen05", TOL_BF16), (torch.bfloat16, "simt", TOL_BF16),
                                            (torch.float32, "auto", TOL_F32)])
@pytest.mark.parametrize("causal,window", [(False, None), (True, None), (True, 90)])
@pytest.mark.parametrize("bh,nq,nk,dqk,dv", [(2, 256, 384, 64, 128), (2, 384, 384, 128, 64), (1, 200, 328, 64, 128),
                                             (3, 130, 259, 128, 64)])
def test_value_head_dim_differs_from_query_key_head_dim(bh, nq, nk, dqk, dv, causal, window, dtype, impl, tol):
    """d_v != d_qk: V, O, dO, ddV (and the results dV2, ddO) have a head dim of their own, as in the
    reference's maths (jax_refs/flash_impl.py:381-389 uses d_in = 256, d_out = 512; its Triton
    operator cannot, fhog/triton_bwdbwd.py:577).  Operator, row statistics, forward and first
    backward against the oracle, which takes any two dims."""
    import fhob
    import math
    wl = math.inf if window is None else window
    x = _two_dim_inputs(bh, nq, nk, dqk, dv, seed=411)
    scale = dqk ** -0.5
    ref = O.bwdbwd_closed_form(*x.values(), scale, causal, sliding_window_length=wl)
    assert ref[2].shape == (bh, nk, dv) and ref[3].shape == (bh, nq, dv)
    o_ref = O.attn_fwd(x["q"], x["k"], x["v"], scale, causal, sliding_window_length=wl)
    l_ref = O.attn_lse(x["q"], x["k"], scale, causal, sliding_window_length=wl)
    dev = {k: v.to(dtype).cuda() for k, v in x.items()}
    kw = dict(is_causal=causal, sliding_window=window, impl=impl)
    args = (dev["q"], dev["k"], dev["v"], o_ref.to(dtype).cuda(), dev["do"], dev["ddq"], dev["ddk"], dev["ddv"],
            l_ref.float().cuda(), scale)
    got = fhob.flash_bwdbwd(*args, check=True, **kw)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert g.shape == r.shape and O.rel_err(g, r) < tol, n
    if window is None:
        sd, sdd, sb = O.bwdbwd_row_stats(*x.values(), scale, causal)
        for fused in ((False, True) if impl != "auto" else (False,)):
            res = fhob.run_passes(*args, is_causal=causal, impl=impl, upto=2, fused12=fused)
            assert res["status"] == 0
            assert O.rel_err(res["d"], sd) < max(tol, 5e-3 if dtype != torch.float32 else 0)
            assert O.rel_err(res["dd"], sdd) < tol and O.rel_err(res["b"], sb) < tol
    if dtype != torch.float32 and impl == "tcgen05":
        got = fhob.flash_bwdbwd(*args[:3], None, *args[4:], check=True, **kw)     # D from the sweep
        for n, g, r in zip(OUT_NAMES, got, ref):
            assert O.rel_err(g, r) < tol, n
    # the producers either side: same kernel family as the operator
    fkw = dict(kw)
    o, lse = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, **fkw)
    assert o.shape == (bh, nq, dv) and O.rel_err(o, o_ref) < tol and O.rel_err(lse, l_ref) < 1e-5
    first = fhob.attention_backward(dev["q"], dev["k"], dev["v"], o, dev["do"], lse, scale, **fkw)
    first_ref = O.attn_bwd(x["q"], x["k"], x["v"], x["do"], scale, causal, sliding_window_length=wl)
    for n, g, r in zip(("dq", "dk", "dv"), first, first_ref):
        assert g.shape == r.shape and O.rel_err(g, r) < tol, n


def test_two_head_dims_through_autograd_and_host_buffers():
    """fhob.attention differentiated twice with d_v != d_qk, and the host-buffer path of the operator."""
    import fhob
    x = _two_dim_inputs(2, 192, 320, 128, 64, seed=413)
    scale = 128 ** -0.5
    ref = O.bwdbwd_autograd(*x.values(), scale, True)
    q, k, v, do = (x[n].bfloat16().cuda().requires_grad_(True) for n in ("q", "k", "v", "do"))
    out = fhob.attention(q, k, v, scale, is_causal=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), do, create_graph=True)
    cot = tuple(x[n].bfloat16().cuda() for n in ("ddq", "ddk", "ddv"))
    got = torch.autograd.grad((dq, dk, dv), (q, k, v, do), cot)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert g.shape == r.shape and O.rel_err(g, r) < TOL_BF16, n
    o = O.attn_fwd(x["q"], x["k"], x["v"], scale, True).bfloat16()
    lse = O.attn_lse(x["q"], x["k"], scale, True).float()
    host = [x[n].bfloat16() for n in ("q", "k", "v")] + [o] + [x[n].bfloat16() for n in ("do", "ddq", "ddk", "ddv")]
    got = fhob.flash_bwdbwd(*host, lse, scale, is_causal=True)
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert g.device.type == "cpu" and g.shape == r.shape and O.rel_err(g, r) < TOL_BF16, n


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("bh,nq,nk,dqk,dv", [(2, 256, 384, 32, 32), (2, 200, 328, 96, 96), (1, 384, 384, 80, 40),
                                             (2, 130, 259, 8, 120), (1, 256, 256, 104, 128), (2, 192, 320, 64, 48)])
def test_head_dims_that_are_not_64_or_128_on_the_tensor_cores(bh, nq, nk, dqk, dv, causal):
    """Any head dims up to 128 that keep rows 16-byte aligned (multiples of 8) run on the tensor-core
    kernels: the TMA boxes reach past the end of a row and are zero-filled there.  Operator (with
    and without the saved output), forward and first backward against the oracle."""
    import fhob
    x = _two_dim_inputs(bh, nq, nk, dqk, dv, seed=431)
    scale = dqk ** -0.5
    ref = O.bwdbwd_closed_form(*x.values(), scale, causal)
    o_ref = O.attn_fwd(x["q"], x["k"], x["v"], scale, causal)
    l_ref = O.attn_lse(x["q"], x["k"], scale, causal)
    dev = {k: v.bfloat16().cuda() for k, v in x.items()}
    kw = dict(is_causal=causal, impl="tcgen05")
    args = (dev["q"], dev["k"], dev["v"], o_ref.bfloat16().cuda(), dev["do"], dev["ddq"], dev["ddk"], dev["ddv"],
            l_ref.float().cuda(), scale)
    for a in (args, args[:3] + (None,) + args[4:]):
        got = fhob.flash_bwdbwd(*a, check=True, **kw)
        for n, g, r in zip(OUT_NAMES, got, ref):
            assert g.shape == r.shape and O.rel_err(g, r) < TOL_BF16, n
    o, lse = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, check=True, **kw)
    assert o.shape == (bh, nq, dv) and O.rel_err(o, o_ref) < TOL_BF16 and O.rel_err(lse, l_ref) < 1e-5
    first = fhob.attention_backward(dev["q"], dev["k"], dev["v"], o, dev["do"], lse, scale, **kw)
    first_ref = O.attn_bwd(x["q"], x["k"], x["v"], x["do"], scale, causal)
    for n, g, r in zip(("dq", "dk", "dv"), first, first_ref):
        assert g.shape == r.shape and O.rel_err(g, r) < TOL_BF16, n


def _as_views(x, b, h, kind):
    """The same values as `x` ((b*h, n, d) tensors) behind non-contiguous memory layouts."""
    out = {}
    for n, t in x.items():
        bh, rows, d = t.shape
        t4 = t.reshape(b, h, rows, d)
        if kind == "bnhd":          # (B, N, H, D) memory seen as (B, H, N, D)
            out[n] = t4.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
        elif kind == "padded":      # rows with padding behind them (a slice of a wider projection), folded 3-D
            wide = torch.zeros(bh, rows, d + 24, dtype=t.dtype, device=t.device)
            wide[..., :d] = t
            out[n] = wide[..., :d]
        elif kind == "hbnd":        # (H, B, N, D) memory seen as (B, H, N, D)
            out[n] = t4.permute(1, 0, 2, 3).contiguous().permute(1, 0, 2, 3)
        assert not out[n].is_contiguous() and torch.equal(out[n].reshape(bh, rows, d), t)
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kind", ["bnhd", "padded", "hbnd"])
def test_views_are_read_in_place(kind, dtype):
    """Non-contiguous inputs (the reference passes every tensor's strides to its kernels,
    fhog/triton_bwdbwd.py:594-610): read through tensor maps without a copy, same bits as the
    contiguous call, for the operator, the forward and the first backward."""
    import fhob
    from fhob.ops import _Problem
    b, h, nq, nk, d = 2, 3, 200, 328, 64
    x = make_inputs(b * h, nq, nk, d, seed=451, dtype=dtype, device="cuda")
    scale = d ** -0.5
    o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], scale, is_causal=True)
    args = (x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, scale)
    want = fhob.flash_bwdbwd(*args, is_causal=True, check=True)
    xv = _as_views(dict(x, o=o), b, h, kind)
    lse_v = lse if kind == "padded" else lse.reshape(b, h, nq)
    vargs = (xv["q"], xv["k"], xv["v"], xv["o"], xv["do"], xv["ddq"], xv["ddk"], xv["ddv"], lse_v, scale)
    prob = _Problem(*vargs, True, "auto")
    assert prob.layout is not None and prob.p.q == xv["q"].data_ptr()       # the caller's memory, no copy
    from fhob import _lib
    import ctypes as C
    assert _lib.load().fhob_bwdbwd(C.byref(prob.p), C.c_void_p(prob.stream)) == 0   # the library takes the layout
    assert prob.status() == 0
    for n, g, w in zip(OUT_NAMES, prob.outputs(), want):
        assert torch.equal(g.reshape(w.shape), w), n
    got = fhob.flash_bwdbwd(*vargs, is_causal=True, check=True)
    for n, g, w in zip(OUT_NAMES, got, want):
        assert g.is_contiguous() and torch.equal(g.reshape(w.shape), w), n
    o2, lse2 = fhob.attention_forward(xv["q"], xv["k"], xv["v"], scale, is_causal=True, check=True)
    assert torch.equal(o2.reshape(o.shape), o) and torch.equal(lse2.reshape(lse.shape), lse)
    first_w = fhob.attention_backward(x["q"], x["k"], x["v"], o, x["do"], lse, scale, is_causal=True)
    first = fhob.attention_backward(xv["q"], xv["k"], xv["v"], xv["o"], xv["do"], lse_v, scale, is_causal=True)
    for g, w in zip(first, first_w):
        assert torch.equal(g.reshape(w.shape), w)
    # the CUDA-core kernels do not take views: the wrapper copies, results unchanged
    sim_w = fhob.flash_bwdbwd(*args, is_causal=True, impl="simt", check=True)
    sim = fhob.flash_bwdbwd(*vargs, is_causal=True, impl="simt", check=True)
    for g, w in zip(sim, sim_w):
        assert torch.equal(g.reshape(w.shape), w)


def test_preallocated_outputs_and_workspace():
    """out= and workspace=: the call writes into the caller's tensors and allocates nothing."""
    import fhob
    from fhob import _lib
    x = make_inputs(3, 256, 320, 128, seed=181, dtype=torch.bfloat16, device="cuda")
    scale = 128 ** -0.5
    o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], scale, is_causal=True)
    args = (x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, scale)
    ref = fhob.flash_bwdbwd(*args, is_causal=True, check=True)
    out = (torch.empty_like(x["q"]), torch.empty_like(x["k"]), torch.empty_like(x["k"]), torch.empty_like(x["q"]))
    ws = torch.empty(_lib.load().fhob_workspace_bytes(3, 256), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    got = fhob.flash_bwdbwd(*args, is_causal=True, out=out, workspace=ws)
    after = torch.cuda.memory_stats()["allocation.all.allocated"]
    torch.cuda.synchronize()
    assert after == before                      # no tensor was allocated by the call
    for g, o_t, r in zip(got, out, ref):
        assert g.data_ptr() == o_t.data_ptr() and torch.equal(g, r)
    with pytest.raises(ValueError):
        fhob.flash_bwdbwd(*args, is_causal=True, out=out[:3])
    with pytest.raises(ValueError):
        fhob.flash_bwdbwd(*args, is_causal=True, out=(out[0], out[1], out[2], out[3].float()))
    with pytest.raises(ValueError):
        fhob.flash_bwdbwd(*args, is_causal=True, workspace=ws[:100])


def test_custom_op_eager_and_compiled():
    """torch.ops.fhob.bwdbwd equals the Python entry point, and a function that calls it compiles
    with fullgraph=True (as the reference's entry point is compiled, fhog/triton_bwdbwd.py:557) and
    reproduces the eager results bit for bit."""
    import fhob
    x = make_inputs(2, 256, 384, 128, seed=191, dtype=torch.bfloat16, device="cuda")
    scale = 128 ** -0.5
    o, lse = fhob.attention_forward(x["q"], x["k"], x["v"], scale, is_causal=True)
    args = (x["q"], x["k"], x["v"], o, x["do"], x["ddq"], x["ddk"], x["ddv"], lse, scale)
    ref = fhob.flash_bwdbwd(*args, is_causal=True, check=True)
    got = torch.ops.fhob.bwdbwd(*args, True, 0)
    for g, r in zip(got, ref):
        assert torch.equal(g, r)

    def step(*a):
        dq2, dk2, dv2, ddo = torch.ops.fhob.bwdbwd(*a, True, 0)
        return dq2 + 0, dk2, dv2, ddo

    compiled = torch.compile(step, fullgraph=True, dynamic=False, backend="aot_eager")
    out = compiled(*args)
    for g, r in zip(out, ref):
        assert torch.equal(g, r)


@pytest.mark.parametrize("nq,nk,d,causal", [(1, 300, 64, False), (3, 3, 128, True), (130, 131, 128, True),
                                            (257, 190, 64, False), (99, 250, 128, True)])
def test_tensor_core_path_takes_any_query_length(nq, nk, d, causal):
    """Query lengths that are not multiples of four (or of anything): the per-head row vectors are
    padded inside the workspace, the tensors themselves are dense."""
    x = make_inputs(3, nq, nk, d, seed=201, dtype=torch.float64)
    got, ref, _ = _run(x, d ** -0.5, causal, torch.bfloat16, "tcgen05")
    for n, g, r in zip(OUT_NAMES, got, ref):
        assert O.rel_err(g, r) < TOL_BF16, n
    res, _, (sd, sdd, sb) = _run(x, d ** -0.5, causal, torch.bfloat16, "tcgen05", upto=2, fused12=True)
    assert O.rel_err(res["d"], sd) < TOL_BF16 and O.rel_err(res["dd"], sdd) < TOL_BF16
    assert O.rel_err(res["b"], sb) < TOL_BF16


@pytest.mark.parametrize("bh,nq,nk,d,causal,window", [(3, 217, 273, 128, True, 1), (1, 267, 1, 64, False, None)])
def test_single_visible_key_gives_vanishing_second_order_terms(bh, nq, nk, d, causal, window):
    """When every query sees exactly one key the softmax is constant: dQ2, dK2 and dV2 are exactly
    zero in the oracle and ddO = ddV of that key.  The kernels must return rounding noise only
    (a relative error is undefined here)."""
    import fhob
    import math
    w = math.inf if window is None else window
    x = make_inputs(bh, nq, nk, d, seed=211, dtype=torch.float64)
    x = {k: v.half().double() for k, v in x.items()}
    scale = d ** -0.5
    ref = O.bwdbwd_closed_form(*x.values(), scale, causal, sliding_window_length=w)
    dev = {k: v.half().cuda() for k, v in x.items()}
    kw = dict(is_causal=causal, sliding_window=window, impl="tcgen05")
    o, lse = fhob.attention_forward(dev["q"], dev["k"], dev["v"], scale, **kw)
    got = fhob.flash_bwdbwd(dev["q"], dev["k"], dev["v"], o, dev["do"], dev["ddq"], dev["ddk"], dev["ddv"], lse,
                            scale, check=True, **kw)
    for n, g, r in zip(OUT_NAMES[:3], got[:3], ref[:3]):
        assert r.abs().max() < 1e-12 and g.double().abs().max() < 1e-4, n
    assert O.rel_err(got[3], ref[3]) < 1e-3
