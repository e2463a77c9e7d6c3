"""Parity at the full benchmark sizes, where the CPU oracle would take minutes: the results
are checked through properties that do not depend on the size — a checksum of checksums (row
sums and column sums of the whole output against float64 products of the operand sums, exact
for the integer triples), exact spot values, whole-output comparison with an fp32 matmul for
the float triples, and pack -> unpack round trips. Inputs are seeded and synthetic."""
import numpy as np
import pytest

from iree_b200 import abi

pytestmark = pytest.mark.gpu

FLOAT_TOL = 1e-3  # relative Frobenius / relative checksum error allowed for f16 and bf16


def _mmt4d(flags, M, N, K, M0, N0, K0, lhs, rhs, out):
    import torch
    from iree_b200 import ukernel as uk
    p = abi.Mmt4dParams()
    p.lhs_buffer, p.rhs_buffer, p.out_buffer = lhs.data_ptr(), rhs.data_ptr(), out.data_ptr()
    p.M, p.N, p.K, p.M0, p.N0, p.K0, p.flags = M, N, K, M0, N0, K0, flags
    p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K * M0 * K0, K * N0 * K0, N * M0 * N0
    n = uk.mmt4d_workspace_size(p)
    ws = torch.empty(max(n, 1), dtype=torch.uint8, device="cuda")
    path = uk.mmt4d_path(p, True)
    uk.mmt4d(p, workspace=ws)
    torch.cuda.synchronize()
    assert uk.device_status() == (0, 0)
    return path


def _logical(t, T1, K1, T0, K0):
    """[T1][K1][T0][K0] tiled operand -> logical [T1*T0][K1*K0] matrix (a view-copy)."""
    return t.view(T1, K1, T0, K0).permute(0, 2, 1, 3).reshape(T1 * T0, K1 * K0)


def _logical_out(t, M1, N1, M0, N0):
    return t.view(M1, N1, M0, N0).permute(0, 2, 1, 3).reshape(M1 * M0, N1 * N0)


def test_s8_prefill_size_checksums_are_exact():
    """s8s8s32, 8192 x 28672 x 8192 in 16x16x2 tiles: every row sum and column sum of the
    int32 output equals the float64 product of the operand with the other operand's sums
    (all values stay below 2^53, so float64 is exact), and 256 sampled outputs are exact."""
    import torch
    M1, N1, K1 = 512, 1792, 4096
    g = torch.Generator(device="cuda").manual_seed(11)
    lhs = torch.randint(-128, 128, (M1 * K1 * 32,), generator=g, device="cuda", dtype=torch.int8)
    rhs = torch.randint(-128, 128, (N1 * K1 * 32,), generator=g, device="cuda", dtype=torch.int8)
    out = torch.full((M1 * N1 * 256,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    path = _mmt4d(abi.MMT4D_S8S8S32, M1, N1, K1, 16, 16, 2, lhs, rhs, out)
    assert path == abi.PATH_TCGEN05_RETILE
    A = _logical(lhs, M1, K1, 16, 2)
    B = _logical(rhs, N1, K1, 16, 2)
    C = _logical_out(out, M1, N1, 16, 16)
    row_sums = C.sum(dim=1, dtype=torch.int64)
    col_sums = C.sum(dim=0, dtype=torch.int64)
    b_sum = B.sum(dim=0, dtype=torch.int64).double()           # [K]
    a_sum = A.sum(dim=0, dtype=torch.int64).double()           # [K]
    want_rows = torch.zeros(A.shape[0], dtype=torch.float64, device="cuda")
    for i in range(0, A.shape[0], 1024):                       # bounded float64 temporaries
        want_rows[i:i + 1024] = A[i:i + 1024].double() @ b_sum
    want_cols = torch.zeros(B.shape[0], dtype=torch.float64, device="cuda")
    for i in range(0, B.shape[0], 1024):
        want_cols[i:i + 1024] = B[i:i + 1024].double() @ a_sum
    assert torch.equal(row_sums, want_rows.long())
    assert torch.equal(col_sums, want_cols.long())
    rng = np.random.default_rng(5)
    for m, n in zip(rng.integers(0, A.shape[0], 256), rng.integers(0, B.shape[0], 256)):
        want = int((A[m].long() * B[n].long()).sum())
        assert int(C[m, n]) == want


def test_bf16_headline_size_against_fp32_matmul():
    """bf16bf16f32 at the headline size: row and column checksums within tolerance of float64
    products of operand sums, and four 256 x 256 output blocks within 1e-3 (relative Frobenius)
    of an fp32 matmul of the same bf16 values."""
    import torch
    M1, N1, K1 = 512, 1792, 4096
    g = torch.Generator(device="cuda").manual_seed(12)
    lhs = torch.randn(M1 * K1 * 32, generator=g, device="cuda").to(torch.bfloat16)
    rhs = (torch.randn(N1 * K1 * 32, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.full((M1 * N1 * 256,), float("nan"), dtype=torch.float32, device="cuda")
    _mmt4d(abi.MMT4D_BF16BF16F32, M1, N1, K1, 16, 16, 2, lhs, rhs, out)
    assert not bool(torch.isnan(out).any())
    A = _logical(lhs, M1, K1, 16, 2)
    B = _logical(rhs, N1, K1, 16, 2)
    C = _logical_out(out, M1, N1, 16, 16)
    want_rows = A.double() @ B.double().sum(dim=0)
    got_rows = C.double().sum(dim=1)
    assert float((got_rows - want_rows).norm() / want_rows.norm()) <= FLOAT_TOL
    want_cols = B.double() @ A.double().sum(dim=0)
    got_cols = C.double().sum(dim=0)
    assert float((got_cols - want_cols).norm() / want_cols.norm()) <= FLOAT_TOL
    for m0, n0 in [(0, 0), (8192 - 256, 28672 - 256), (4096, 1024), (512, 20480)]:
        want = A[m0:m0 + 256].float() @ B[n0:n0 + 256].float().t()
        got = C[m0:m0 + 256, n0:n0 + 256]
        assert float((got - want).norm() / want.norm()) <= FLOAT_TOL


def test_f16_accumulate_4096_whole_output():
    """f16f16f32 | ACCUMULATE, 4096^3 in 16x16x1 tiles: the whole output against
    accumulator + fp32 matmul."""
    import torch
    M1 = N1 = 256
    K1 = 4096
    g = torch.Generator(device="cuda").manual_seed(13)
    lhs = torch.randn(M1 * K1 * 16, generator=g, device="cuda").to(torch.float16)
    rhs = torch.randn(N1 * K1 * 16, generator=g, device="cuda").to(torch.float16)
    acc = torch.randn(M1 * N1 * 256, generator=g, device="cuda")
    out = acc.clone()
    _mmt4d(abi.MMT4D_F16F16F32 | abi.MMT4D_ACCUMULATE, M1, N1, K1, 16, 16, 1, lhs, rhs, out)
    A = _logical(lhs, M1, K1, 16, 1)
    B = _logical(rhs, N1, K1, 16, 1)
    torch.backends.cuda.matmul.allow_tf32 = False
    want = _logical_out(acc, M1, N1, 16, 16) + A.float() @ B.float().t()
    got = _logical_out(out, M1, N1, 16, 16)
    assert float((got - want).norm() / want.norm()) <= FLOAT_TOL


def test_s16u4_decode_gemv_whole_output_exact():
    """s16u4s32 1x32x8, N1 = 448, K1 = 512 (1 x 14336 x 4096): all 14336 outputs equal the
    int64 dot products reduced modulo 2^32."""
    import torch
    N1, K1 = 448, 512
    g = torch.Generator(device="cuda").manual_seed(14)
    lhs = torch.randint(-32768, 32768, (K1 * 8,), generator=g, device="cuda", dtype=torch.int16)
    rhs = torch.randint(0, 256, (N1 * K1 * 128,), generator=g, device="cuda", dtype=torch.uint8)
    out = torch.zeros(N1 * 32, dtype=torch.int32, device="cuda")
    path = _mmt4d(abi.MMT4D_S16U4S32, 1, N1, K1, 1, 32, 8, lhs, rhs, out)
    assert path == abi.PATH_GEMV
    b = rhs.view(N1, K1, 32, 4).long()                 # bytes: low nibble = even k0
    w = torch.stack([b & 15, b >> 4], dim=-1).reshape(N1, K1, 32, 8)   # [n1][k1][n0][k0]
    x = lhs.view(K1, 8).long()
    want = (w * x[None, :, None, :]).sum(dim=(1, 3)).reshape(-1)
    want = ((want + 2 ** 31) % 2 ** 32 - 2 ** 31).int()
    assert torch.equal(out, want)


@pytest.mark.parametrize("rows,cols", [(8192, 8192), (8185, 8190)], ids=["exact", "padded"])
def test_pack_then_unpack_is_the_identity_at_8192(rows, cols):
    """f32 rows x cols -> [512][512][16][16] -> rows x cols: bit-exact round trip; with a
    ragged shape the padding holds the padding value and never reaches the result."""
    import torch
    from iree_b200 import ukernel as uk
    g = torch.Generator(device="cuda").manual_seed(15)
    src = torch.randn(rows * cols, generator=g, device="cuda")
    packed = torch.full((512 * 512 * 256,), 7.0, device="cuda")
    back = torch.full((rows * cols,), -1.0, device="cuda")
    p = abi.PackParams()
    p.in_buffer, p.out_buffer = src.data_ptr(), packed.data_ptr()
    p.in_size0, p.in_size1, p.in_stride0, p.in_stride1 = rows, cols, cols, 1
    p.out_size0, p.out_size1, p.out_size2, p.out_size3 = 512, 512, 16, 16
    p.out_stride1, p.out_stride0 = 256, 512 * 256
    p.padding_value = 0x7FC00000          # a NaN pattern: bits must be copied, not converted
    p.flags = abi.PACK_F32F32
    uk.pack(p)
    u = abi.UnpackParams()
    u.in_buffer, u.out_buffer = packed.data_ptr(), back.data_ptr()
    u.in_size0, u.in_size1, u.in_size2, u.in_size3 = 512, 512, 16, 16
    u.in_stride1, u.in_stride0 = 256, 512 * 256
    u.out_size0, u.out_size1, u.out_stride0, u.out_stride1 = rows, cols, cols, 1
    u.flags = abi.UNPACK_F32F32
    uk.unpack(u)
    torch.cuda.synchronize()
    assert torch.equal(back.view(torch.int32), src.view(torch.int32))
    tiles = packed.view(512, 512, 16, 16).permute(0, 2, 1, 3).reshape(8192, 8192).view(torch.int32)
    assert torch.equal(tiles[:rows, :cols], src.view(rows, cols).view(torch.int32))
    if rows < 8192:
        assert bool((tiles[rows:, :] == 0x7FC00000).all())
        assert bool((tiles[:, cols:] == 0x7FC00000).all())


def test_fused_matmul_s8_full_size_checksums_are_exact():
    """iree_uk_b200_matmul, s8, 8192 x 28672 x 8192 row-major: exact row and column sums."""
    import torch
    from iree_b200 import ukernel as uk
    M, N, K = 8192, 28672, 8192
    g = torch.Generator(device="cuda").manual_seed(16)
    A = torch.randint(-128, 128, (M, K), generator=g, device="cuda", dtype=torch.int8)
    B = torch.randint(-128, 128, (K, N), generator=g, device="cuda", dtype=torch.int8)
    C = torch.full((M, N), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    p = abi.MatmulParams()
    p.lhs_buffer, p.rhs_buffer, p.out_buffer = A.data_ptr(), B.data_ptr(), C.data_ptr()
    p.lhs_stride0, p.rhs_stride0, p.out_stride0 = K, N, N
    p.M, p.N, p.K, p.flags = M, N, K, abi.MMT4D_S8S8S32
    ws = torch.empty(uk.matmul_workspace_size(p), dtype=torch.uint8, device="cuda")
    uk.matmul(p, ws)
    torch.cuda.synchronize()
    assert uk.device_status() == (0, 0)
    b_sum = B.sum(dim=1, dtype=torch.int64).double()           # [K]
    a_sum = A.sum(dim=0, dtype=torch.int64).double()           # [K]
    want_rows = torch.cat([A[i:i + 1024].double() @ b_sum for i in range(0, M, 1024)])
    want_cols = torch.cat([a_sum @ B[:, j:j + 1024].double() for j in range(0, N, 1024)])
    assert torch.equal(C.sum(dim=1, dtype=torch.int64), want_rows.long())
    assert torch.equal(C.sum(dim=0, dtype=torch.int64), want_cols.long())
