"""The arithmetic of the integer tensor-core kernel (minit_b200/csrc/qgemm_mid.cu), restated exactly on the host: per
row and per 128 values of k a power-of-two scale brings the block maximum into [2^13, 2^14), the scaled activations are
rounded to integers and split into two signed-byte limbs, the products with the unsigned weights are exact integer sums,
and every k-block is folded in fp32 as ``s * 2^-e * (V - (z + 1) * sum(x'))``.  What this checks without a GPU: the limbs
fit the tensor core's signed bytes and reconstruct the integer; the block fixed point stays inside the 1e-2 * rms bound
of the GEMM tests for activations with an outlier in EVERY block (up to 10 000 times the typical value), for heavy
tails, for rows of very different magnitude and for values below the fp16 normal range."""
import numpy as np
import pytest
import torch

from oracle import qlinear_oracle as O


def block_fixed_point(block: np.ndarray):
    """block [M, 128] float64 -> (x' int64 [M, 128], e int [M]) as xprep_kernel computes them"""
    amax = np.abs(block).max(axis=1).astype(np.float32)
    e = np.zeros(len(amax), dtype=np.int64)
    ok = (amax > 0) & (amax < 3.0e38)
    exponent = ((amax.view(np.uint32) >> 23) & 0xff).astype(np.int64) - 127       # the float's exponent field, as the kernel reads it
    e[ok] = 13 - exponent[ok]
    e = np.clip(e, -100, 100)
    scaled = np.clip(block.astype(np.float32) * np.exp2(e).astype(np.float32)[:, None], -16384.0, 16384.0)
    return np.rint(scaled).astype(np.int64), e


def limbs(xi: np.ndarray):
    lo = ((xi + 128) & 255) - 128
    hi = (xi - lo) >> 8
    return hi, lo


def emulate(x: torch.Tensor, q: np.ndarray, z: np.ndarray, scales: torch.Tensor, group_size: int) -> torch.Tensor:
    xf = x.double().numpy()
    m, k = xf.shape
    acc = np.zeros((m, q.shape[1]), dtype=np.float32)
    for kb in range(k // 128):
        xi, e = block_fixed_point(xf[:, kb * 128:(kb + 1) * 128])
        hi, lo = limbs(xi)
        assert hi.min() >= -128 and hi.max() <= 127 and lo.min() >= -128 and lo.max() <= 127
        assert np.array_equal(256 * hi + lo, xi)
        w = q[kb * 128:(kb + 1) * 128].astype(np.int64)
        v = 256 * (hi @ w) + lo @ w                                               # the two MMAs of a k-block, exact 32-bit sums
        assert np.abs(hi @ w).max() < 2 ** 31 and np.abs(lo @ w).max() < 2 ** 31
        g = (kb * 128) // group_size
        term = (v - (z[g].astype(np.int64) + 1)[None, :] * xi.sum(axis=1)[:, None]).astype(np.float32)
        acc += (scales[g].float().numpy()[None, :] * np.exp2(-e).astype(np.float32)[:, None]) * term
    return torch.from_numpy(acc).to(x.dtype)


def _ratio(x: torch.Tensor, c, group_size=128):
    w = O.dequantize(c["q"], c["g_idx"].numpy(), c["z"], c["scales"])
    ref = O.qlinear(x, w)
    ok, err, bound = O.tolerance_ok(emulate(x, c["q"], c["z"], c["scales"], group_size), ref, 1e-2)
    return err / bound


@pytest.mark.parametrize("outlier", [1, 30, 1000, 10000])
def test_an_outlier_in_every_block(outlier):
    for bits in (4, 8):
        c = O.make_gptq_case(2048, 128, 3, bits=bits, seed=outlier % 97 + bits)
        g = torch.Generator().manual_seed(outlier)
        x = torch.randn((3, 2048), generator=g)
        where = torch.randint(0, 128, (16,), generator=g) + torch.arange(16) * 128
        x[:, where] *= outlier
        x = x * (50.0 / x.abs().max())                                           # keep fp16 in range
        assert _ratio(x.half(), c) < 0.5                                         # half of the GEMM tests' bound


def test_heavy_tails_and_mixed_rows():
    c = O.make_gptq_case(4096, 128, 5, bits=4, seed=9)
    x = torch.from_numpy(np.random.default_rng(5).standard_t(2, size=(5, 4096))).float().clamp(-6e4, 6e4)
    x[1] *= 1e-3
    x[2] = 0
    x[3, ::2] *= 1e-4
    for row in range(5):
        if row == 2:
            assert emulate(x[2:3].half(), c["q"], c["z"], c["scales"], 128).abs().max() == 0
        else:
            assert _ratio(x[row:row + 1].half(), c) < 0.5, row


def test_values_below_the_fp16_normal_range_keep_their_bits():
    """a block whose largest value is an fp16 subnormal is scaled up like any other: nothing is flushed"""
    x = torch.zeros((1, 128), dtype=torch.float16)
    x[0, 3], x[0, 77] = 2.0 ** -24, 3 * 2.0 ** -24
    xi, e = block_fixed_point(x.double().numpy())
    assert xi[0, 3] * 3 == xi[0, 77] and xi[0, 77] >= 2 ** 13 and int(e[0]) == 13 + 23
