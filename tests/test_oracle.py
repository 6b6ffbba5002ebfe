"""Pin the CPU oracle (oracle/block_fp8_ref.py) against outputs of the reference's own
functions, stored in tests/golden/ by tests/golden/make_golden.py."""
import numpy as np
import pytest
import torch

from oracle import block_fp8_ref as oracle

N_CASES = 8


def _case(golden, i):
    g = lambda key: golden[f"c{i}_{key}"]
    return g("meta"), g("A"), g("B"), g("As"), g("Bs"), g("ref32"), g("ref16_bits")


def test_e4m3_decode_matches_torch_for_all_bytes():
    b = torch.arange(256, dtype=torch.uint8)
    want = b.view(torch.float8_e4m3fn).float().numpy()
    got = oracle.e4m3_decode(b.numpy())
    assert np.array_equal(np.isnan(want), np.isnan(got))
    assert np.array_equal(want[~np.isnan(want)], got[~np.isnan(got)])


def test_e4m3_encode_matches_torch_cast():
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 100,
        rng.standard_normal(20000).astype(np.float32) * 0.01,
        np.linspace(-448, 448, 8193, dtype=np.float32),
        np.array([0.0, -0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10, 464.0, 1e-12], np.float32),
    ])
    x = x[np.abs(x) <= 464]         # beyond the last rounding boundary torch saturates/NaNs: unused
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = oracle.e4m3_encode(x)
    ok = (want == got) | ((want & 0x7F == 0) & (got & 0x7F == 0))   # +-0 both fine
    assert ok.all(), (x[~ok][:8], want[~ok][:8], got[~ok][:8])


def test_bf16_round_matches_torch():
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(100000) * 10 ** rng.uniform(-6, 6, 100000)).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.bf16_bits(x), want)


@pytest.mark.parametrize("i", range(N_CASES))
def test_gemm_fp32_equals_reference_output(golden, i):
    meta, A, B, As, Bs, ref32, ref16_bits = _case(golden, i)
    got = oracle.gemm_fp32(A, B, As, Bs)
    # Same arithmetic (fp32 dequant, fp32 sgemm) but a different BLAS blocking than torch:
    # equal to within a few fp32 ulps of the largest row/column products.
    scale = max(float(np.abs(ref32).max()), 1e-30)
    assert np.abs(got - ref32).max() <= 4e-6 * scale
    # after the bf16 cast of bench.py:30 the two agree except for rare 1-ulp ties
    bits = oracle.bf16_bits(got).astype(np.int32)
    want = ref16_bits.view(np.uint16).astype(np.int32)
    assert (np.abs(bits - want) <= 1).all()
    assert (bits != want).mean() < 2e-3


@pytest.mark.parametrize("i", range(N_CASES))
def test_error_metric_equals_reference_error(golden, i):
    _, A, B, As, Bs, ref32, ref16_bits = _case(golden, i)
    ref16 = (ref16_bits.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    assert oracle.rel_error(ref16, ref32) == pytest.approx(float(golden[f"c{i}_err_bf16"]), rel=1e-6, abs=1e-12)
    noisy = (ref16 * np.float32(1 + 1e-3)).astype(np.float32)
    assert oracle.rel_error(noisy, ref32) == pytest.approx(float(golden[f"c{i}_err_noisy"]), rel=1e-5, abs=1e-12)


@pytest.mark.parametrize("i", range(N_CASES))
def test_quantizer_equals_reference_recipe(golden, i):
    if f"c{i}_x" not in golden:
        pytest.skip("raw inputs stored for the small cases only")
    _, A, B, As, Bs, _, _ = _case(golden, i)
    a_q, a_s = oracle.quantize_activations(golden[f"c{i}_x"], 1e-6)
    b_q, b_s = oracle.quantize_weights(golden[f"c{i}_w"], 1e-6)
    assert np.array_equal(a_s, As) and np.array_equal(b_s, Bs)
    for got, want in ((a_q, A), (b_q, B)):
        same = (got == want) | ((got & 0x7F == 0) & (want & 0x7F == 0))
        assert same.all()


@pytest.mark.parametrize("i", range(N_CASES))
def test_blockwise_order_is_within_tolerance_of_reference(golden, i):
    _, A, B, As, Bs, ref32, _ = _case(golden, i)
    got = oracle.bf16_round(oracle.gemm_blockwise(A, B, As, Bs))
    assert oracle.rel_error(got, ref32) <= 1e-2
    assert oracle.elementwise_violations(got, ref32) == 0


def test_product_quantizer_agrees_with_oracle_quantizer():
    from fp8_gemm_h20_b200 import testing
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(19, 384, generator=gen)
    w = torch.randn(256, 384, generator=gen) * 0.02
    A, As = testing.quantize_activations(x)
    B, Bs = testing.quantize_weights(w)
    a_q, a_s = oracle.quantize_activations(x.numpy())
    b_q, b_s = oracle.quantize_weights(w.numpy())
    assert np.array_equal(As.numpy(), a_s) and np.array_equal(Bs.numpy(), b_s)
    assert np.array_equal(A.view(torch.uint8).numpy() & 0x7F | 0, a_q & 0x7F | 0) or \
        np.array_equal(A.view(torch.uint8).numpy(), a_q)
    assert np.array_equal(B.view(torch.uint8).numpy(), b_q) or \
        ((B.view(torch.uint8).numpy() ^ b_q) & 0x7F == 0).all()


def test_product_torch_reference_agrees_with_oracle():
    from fp8_gemm_h20_b200 import testing
    A, B, As, Bs = testing.make_problem(33, 256, 512, seed=11, mode="cfg0")
    want = oracle.gemm_fp32(A.view(torch.uint8).numpy(), B.view(torch.uint8).numpy(), As.numpy(), Bs.numpy())
    got = testing.reference_fp32(A, B, As, Bs).numpy()
    assert np.abs(got - want).max() <= 4e-6 * np.abs(want).max()


def test_ue8m0_expansion_known_answers():
    """UE8M0 = exponent-only scale, 2^(e-127); 127 -> 1.0, 0 -> 2^-127 (subnormal), 255 -> NaN."""
    from oracle.block_fp8_ref import expand_ue8m0, unpack_ue8m0_words
    e = np.array([0, 1, 120, 126, 127, 128, 134, 254], dtype=np.uint8)
    v = expand_ue8m0(e)
    assert v.dtype == np.float32
    assert v.view(np.uint32).tolist() == [0x00400000] + [int(x) << 23 for x in e[1:]]
    assert v[4] == 1.0 and v[5] == 2.0 and v[3] == 0.5 and v[2] == 2.0 ** -7
    assert np.isnan(expand_ue8m0(np.array([255], dtype=np.uint8))[0])
    words = np.array([[0x7F7E7D7C, 0x01000280 - (1 << 32)]], dtype=np.int64).astype(np.int32)
    assert unpack_ue8m0_words(words).tolist() == [[0x7C, 0x7D, 0x7E, 0x7F, 0x80, 0x02, 0x00, 0x01]]
