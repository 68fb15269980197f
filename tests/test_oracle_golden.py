"""CPU: the oracle against the golden vectors recorded from the reference
itself (tests/golden/make_golden.py), plus the pins the reference's own tests
put on the block-scaled path."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import tcfp_oracle as O
from tests.golden.cases import CAST_CASES, LAYER_CASES, cast_input, layer_inputs
from tests.util import weights

GOLD = np.load(Path(__file__).parent / "golden" / "per_tensor.npz")


def u8(t):
    return t.contiguous().view(torch.uint8).numpy()


def i32(t):
    return t.float().contiguous().view(torch.int32).numpy()


def f32(a):
    return torch.from_numpy(a.copy()).view(torch.float32)


@pytest.mark.parametrize("name", list(CAST_CASES))
def test_casts_match_reference_bits(name):
    seed, shape, dtype = CAST_CASES[name]
    x = cast_input(seed, shape, dtype)
    q, inv = O.to_fp8_e4m3(x)
    assert np.array_equal(u8(q), GOLD[f"cast/{name}/e4m3"]) and np.array_equal(i32(inv), GOLD[f"cast/{name}/e4m3_inv"])
    q, inv = O.to_fp8_e5m2(x)
    assert np.array_equal(u8(q), GOLD[f"cast/{name}/e5m2"]) and np.array_equal(i32(inv), GOLD[f"cast/{name}/e5m2_inv"])
    q, inv = O.to_fp8_e4m3_nf_aware(x)
    assert np.array_equal(u8(q), GOLD[f"cast/{name}/nf_aware"]) and np.array_equal(i32(inv), GOLD[f"cast/{name}/nf_aware_inv"])
    scaled = (x.float() * (448.0 / x.float().abs().max())).clamp(-448, 448)
    rand = O.philox_uniform_packed(seed, 17, scaled.numel()).reshape(scaled.shape)
    assert np.array_equal(u8(O.stochastic_round_to_fp8_e4m3(scaled, rand)), GOLD[f"cast/{name}/sr"])


@pytest.mark.parametrize("name", list(LAYER_CASES))
def test_layer_steps_match_reference(name):
    """Two training steps: error-feedback / delayed-scaling state bit for bit,
    outputs and gradients to 1e-3 relative Frobenius (the reference ran
    ``torch._scaled_mm`` on CPU, the oracle a dequantized FP32 matmul)."""
    cfg = LAYER_CASES[name]
    x, w, b, target = layer_inputs(cfg)
    w = w.clone()
    srr = cfg.get("srr", False)
    state = O.LayerState()
    for step in range(2):
        xin = x.clone()
        y, ctx = O.linear_forward(xin, w, b, state, srr=srr, abd=cfg.get("abd", False),
                                  delayed=cfg.get("delayed", False), hp_grad_weight=cfg.get("hp", False),
                                  seed=cfg["seed"], nf_sigma=3.0 if cfg.get("nf") else None)
        gy = 2.0 * (y - target) / y.numel()
        dx, dw, db = O.linear_backward(ctx, gy)
        pre = f"layer/{name}/step{step}/"
        for key, val in (("y", y), ("dx", dx), ("dw", dw)):
            ref = f32(GOLD[pre + key]).reshape(val.shape)
            assert float((val - ref).norm() / ref.norm()) <= 1e-3, key
        if b is not None:
            ref = f32(GOLD[pre + "db"])
            assert float((db - ref).norm() / ref.norm()) <= 1e-3
        if not srr:
            assert np.array_equal(i32(state.error), GOLD[pre + "ef"]), "error-feedback buffer differs"
        if cfg.get("delayed"):
            assert np.array_equal(i32(state.delayed_amax.reshape(1)), GOLD[pre + "delayed/layer.w_hi"])
            assert np.array_equal(i32(state.ratio.reshape(1)), GOLD[pre + "ratio/layer.ratio"])
        # the same SGD update as the generator, on the golden gradient so that
        # step 2 starts from identical weights
        w = w - 0.05 * f32(GOLD[pre + "dw"]).reshape(w.shape)


def test_philox_known_answers():
    # Random123 known-answer vector for philox4x32-10, counter = key = 0
    assert int(O.philox4x32_10(0, np.array([0], dtype=np.uint64))[0]) == 0x6627E8D5
    u = O.philox_uniform(123, 0, 4096)
    assert float(u.min()) >= 0.0 and float(u.max()) < 1.0 and abs(float(u.mean()) - 0.5) < 0.02
    # offset contract: a shifted window of the same stream
    assert torch.equal(O.philox_uniform(123, 100, 16), O.philox_uniform(123, 0, 116)[100:])
    # high counter word is used
    assert not torch.equal(O.philox_uniform(1, 0, 8), O.philox_uniform(1, 1 << 32, 8))
    # all four output words (Random123 known-answer vector, zero counter and key)
    words = O.philox4x32_10(0, np.array([0], dtype=np.uint64), all_words=True)[:, 0]
    assert [int(w) for w in words] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    # packed per-tensor stream: element j is word j & 3 of call j >> 2, at any offset
    full = O.philox_uniform_packed(77, 0, 64)
    calls = O.philox4x32_10(77, np.arange(16, dtype=np.uint64), all_words=True)
    assert torch.equal(full, torch.from_numpy(O._word_to_uniform(np.ascontiguousarray(calls.T.reshape(-1)))))
    assert torch.equal(full[::4], O.philox_uniform(77, 0, 16))
    for off, n in ((1, 7), (3, 13), (17, 40), (4, 8)):
        assert torch.equal(O.philox_uniform_packed(77, off, n), full[off:off + n])


@pytest.mark.parametrize("bs", [32, 64, 128])
def test_block_dual_equals_two_sequential_quantizes(bs):
    """tests/test_fused_dual_quant.py:80-155, 287-306 of the reference."""
    w = weights(5, 64, 256, outliers=True)
    err = weights(6, 64, 256, std=1e-4)
    hi, lo, eh, el, new_err = O.dual_quantize_block(w, bs, err)
    hi2, eh2 = O.block_quantize(w + err, bs)
    lo2, el2 = O.block_quantize((w + err) - O.block_dequantize(hi2, eh2, bs), bs)
    assert torch.equal(hi.view(torch.uint8), hi2.view(torch.uint8)) and torch.equal(eh, eh2)
    assert torch.equal(lo.view(torch.uint8), lo2.view(torch.uint8))
    keep = el != -128
    assert torch.equal(el[keep], el2[keep])
    # EF formula (tests/test_fused_dual_quant.py:232-250)
    expect = w - O.block_dequantize(hi, eh, bs) - O.block_dequantize(lo, el, bs)
    assert torch.equal(new_err, expect)
    assert eh.shape == (256 // bs, 64) and eh.dtype == torch.int8 and int(eh.min()) >= -126


def test_block_zero_residual_sentinel():
    w = torch.ones(8, 64)          # exactly representable -> zero residual
    hi, lo, eh, el, _ = O.dual_quantize_block(w, 32)
    assert bool((el == -128).all()) and bool((lo.float() == 0).all())
    out = O.block_dual_gemm_nt(*O.block_quantize(torch.ones(4, 64), 32), hi, eh, lo, el, 32)
    assert torch.equal(out, torch.full((4, 8), 64.0))


def test_block_exponent_near_powers_of_two():
    """The float32 log2 of amax/448 rounds to an integer for amax a few ulps
    above 448*2^k; the exponent rule must follow torch, not exact math."""
    for k in range(-50, 100, 7):
        base = np.float32(2.0**k)
        q = (base.view(np.uint32) + np.arange(0, 64, dtype=np.uint32)).view(np.float32)
        e = torch.ceil(torch.log2(torch.from_numpy(q.copy())))
        exact = np.ceil(np.log2(q.astype(np.float64)).astype(np.float32))
        assert np.array_equal(e.numpy(), exact)


def test_srr_block_unbiased():
    """tests/test_fused_dual_quant.py:494-526: relative bias of the mean over
    many draws is small."""
    w = weights(9, 16, 64)
    acc = torch.zeros_like(w)
    n = 300
    for i in range(n):
        hi, lo, eh, el, _ = O.dual_quantize_block(w, 32, srr=True, seed=i)
        acc += O.block_dequantize(hi, eh, 32) + O.block_dequantize(lo, el, 32)
    assert float((acc / n - w).abs().mean() / w.abs().mean()) < 1e-3
