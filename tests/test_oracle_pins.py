"""Pins the CPU oracle (oracle/uk_oracle.c): against the committed golden vectors produced by
the compiled reference ukernels, and — where the compiled reference itself is present —
against it directly on the reference tests' full case lists."""
import numpy as np
import pytest

import oracle
from iree_b200 import abi
from oracle import cases

import golden_util

needs_ref = pytest.mark.skipif(not oracle.ref_available(),
                               reason="compiled reference ukernels not present")


def test_oracle_matches_golden_mmt4d():
    gs = golden_util.load("mmt4d")
    assert len(gs) > 100
    for g in gs:
        out = g.bufs["init"].copy()
        oracle.mmt4d(g.params(g.bufs["lhs"], g.bufs["rhs"], out))
        assert np.array_equal(out, g.bufs["out"]), g.values


def test_oracle_matches_golden_pack():
    gs = golden_util.load("pack")
    assert len(gs) > 50
    for g in gs:
        out = g.bufs["init"].copy()
        oracle.pack(g.params(g.bufs["in"], out))
        assert np.array_equal(out, g.bufs["out"]), g.values


def test_oracle_matches_golden_unpack():
    gs = golden_util.load("unpack")
    assert len(gs) > 20
    for g in gs:
        out = g.bufs["init"].copy()
        oracle.unpack(g.params(g.bufs["in"], out))
        assert np.array_equal(out, g.bufs["out"]), g.values


@needs_ref
def test_oracle_matches_reference_mmt4d_case_list():
    """Whole-buffer equality on tools/mmt4d_test.c's shapes x tiles x narrowed M0 x
    accumulate, against both the ISA-specific and the portable reference code paths."""
    n = 0
    for c in cases.all_mmt4d_cases(cases.MMT4D_TILES + cases.MMT4D_TILES_EXTRA +
                                   cases.MMT4D_TILES_16BIT_OUT):
        want = c.out_init.copy()
        oracle.mmt4d(c.params(c.lhs, c.rhs, want))
        for feat in ("host", "none"):
            got = c.out_init.copy()
            oracle.mmt4d(c.params(c.lhs, c.rhs, got), "ref", feat)
            assert np.array_equal(got, want), (c.label(), feat)
        n += 1
    assert n > 1000


@needs_ref
def test_oracle_matches_reference_pack_unpack_case_lists():
    for c in cases.all_pack_cases():
        a, b = c.out_init.copy(), c.out_init.copy()
        oracle.pack(c.params(c.inp, a))
        oracle.pack(c.params(c.inp, b), "ref")
        assert np.array_equal(a, b), vars(c)
    for c in cases.all_unpack_cases():
        a, b = c.out_init.copy(), c.out_init.copy()
        oracle.unpack(c.params(c.inp, a))
        oracle.unpack(c.params(c.inp, b), "ref")
        assert np.array_equal(a, b), vars(c)


@needs_ref
@pytest.mark.parametrize("t,M0,N0,K0,acc", [(abi.MMT4D_F16F16F32, 16, 16, 1, 1),
                                            (abi.MMT4D_BF16BF16F32, 16, 16, 2, 0)])
def test_oracle_float_normal_close_to_reference(t, M0, N0, K0, acc):
    """N(0,1) operands: the oracle's sequential f32 accumulation and the reference's AVX-512
    paths agree to float round-off (far inside the 1e-3 parity tolerance)."""
    c = cases.Mmt4dCase(t, M0, N0, K0, 8, 8, 256, acc, seed=5, mode="normal", loose=False)
    a, b = c.out_init.copy(), c.out_init.copy()
    oracle.mmt4d(c.params(c.lhs, c.rhs, a))
    oracle.mmt4d(c.params(c.lhs, c.rhs, b), "ref")
    assert cases.rel_frobenius(a.view(np.float32), b.view(np.float32)) < 1e-5


@needs_ref
def test_reference_headline_integer_configs_small():
    """Scaled-down s8s8s32 16x16x2 and s16u4s32 1x32x8 problems with full-range values."""
    for (t, M0, N0, K0, M, N, K) in [(abi.MMT4D_S8S8S32, 16, 16, 2, 8, 8, 64),
                                     (abi.MMT4D_S16U4S32, 1, 32, 8, 1, 14, 64)]:
        c = cases.Mmt4dCase(t, M0, N0, K0, M, N, K, 0, seed=9, mode="normal", loose=False)
        a, b = c.out_init.copy(), c.out_init.copy()
        oracle.mmt4d(c.params(c.lhs, c.rhs, a))
        oracle.mmt4d(c.params(c.lhs, c.rhs, b), "ref")
        assert np.array_equal(a, b)


def test_threaded_driver_matches_single_call():
    for (t, M0, N0, K0, M, N, K) in [(abi.MMT4D_S8S8S32, 16, 16, 2, 13, 5, 9),
                                     (abi.MMT4D_S16U4S32, 1, 32, 8, 1, 11, 7)]:
        c = cases.Mmt4dCase(t, M0, N0, K0, M, N, K, 1, seed=4, loose=False)
        a, b = c.out_init.copy(), c.out_init.copy()
        oracle.mmt4d(c.params(c.lhs, c.rhs, a))
        oracle.mmt4d_threaded(c.params(c.lhs, c.rhs, b), 4, impl="oracle")
        assert np.array_equal(a, b)


def test_matmul_chain_restatement_against_reference_and_plain_matmul():
    """The pack -> mmt4d -> unpack chain (ukernel/tools/e2e_matmul_benchmark.c:173-300) on the
    oracle equals the same chain on the compiled reference and a plain integer matmul, for
    several tile sizes including ones that need padding."""
    rng = np.random.default_rng(5)
    M, N, K = 45, 70, 37
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    b = rng.integers(-128, 128, (K, N), dtype=np.int8)
    c = rng.integers(-1000, 1000, (M, N), dtype=np.int32)
    want = a.astype(np.int32) @ b.astype(np.int32) + c
    impls = ["oracle"] + (["ref"] if oracle.ref_available() else [])
    for impl in impls:
        for tile in [(16, 16, 2), (8, 8, 4), (7, 3, 5)]:
            got = oracle.matmul_chain(a, b, c, abi.MMT4D_S8S8S32, *tile, impl=impl)
            assert np.array_equal(got, want), (impl, tile)
    assert np.array_equal(oracle.matmul_chain(a, b, None, abi.MMT4D_S8S8S32, 16, 16, 2), want - c)
