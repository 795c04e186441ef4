"""GPU parity: pack/unpack, Algorithm 1 and Algorithm 2 kernels against the golden fixtures and the oracle."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from util import MAX_TIE_RATE, code_mismatches

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tq():
    import turboquant_kv.reference as R

    return R


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_pack_unpack_golden(tq, golden):
    g = golden("pack")
    for bits in (1, 2, 3, 4):
        for dim in (8, 20, 32, 64, 100, 128, 256):
            codes, packed = g[f"codes_b{bits}_d{dim}"], g[f"packed_b{bits}_d{dim}"]
            assert np.array_equal(tq.pack_codes(cuda(codes), bits).cpu().numpy(), packed)
            assert np.array_equal(tq.unpack_codes(cuda(packed), bits, dim).cpu().numpy(), codes)


def test_pack_unpack_empty_and_host_tensors(tq):
    assert tq.pack_codes(torch.zeros(0, 64, dtype=torch.uint8, device="cuda"), 4).shape == (0, 32)
    codes = torch.randint(0, 8, (33, 100), dtype=torch.uint8)  # host tensor: staged on the GPU, returned on the host
    packed = tq.pack_codes(codes, 3)
    assert packed.device.type == "cpu" and packed.shape == (33, 39)
    assert torch.equal(tq.unpack_codes(packed, 3, 100), codes)


@pytest.mark.parametrize("dim", [128, 64, 32])
def test_quantize_mse_golden_and_oracle(tq, orc, golden, dim):
    g = golden("mse")
    x = g[f"x_d{dim}"]
    rot = orc.make_rotation_matrix(dim, 42)
    for bits in (1, 2, 3, 4):
        bnd, cent = orc.lloyd_max_codebook(bits, dim)
        packed, norms = tq.quantize_mse(cuda(x), bits, rotation=cuda(rot), codebook=(cuda(bnd), cuda(cent)))
        o_packed, o_norms, rotated = orc.quantize_mse(x, bits, rot, bnd, return_rotated=True)
        rate, _ = code_mismatches(orc, packed.cpu().numpy(), o_packed, rotated, bnd, bits, dim)
        assert rate <= 1e-3
        rate_g, _ = code_mismatches(orc, packed.cpu().numpy(), g[f"packed_b{bits}_d{dim}"], rotated, bnd, bits, dim)
        assert rate_g <= 1e-3
        np.testing.assert_allclose(norms.cpu().numpy(), g[f"norms_b{bits}_d{dim}"], rtol=2e-6)
        recon = tq.dequantize_mse(cuda(g[f"packed_b{bits}_d{dim}"]), cuda(g[f"norms_b{bits}_d{dim}"]), bits, dim,
                                  rotation=cuda(rot), codebook=(cuda(bnd), cuda(cent)))
        ref = g[f"recon_b{bits}_d{dim}"]
        np.testing.assert_allclose(recon.cpu().numpy()[:64], ref, rtol=1e-4, atol=1e-5 * np.abs(ref).max())


def test_quantize_mse_full_unit_sphere_config(tq, orc, golden):
    """65,536 x 128, 4 bits, unit-norm rows: mismatch rate against the oracle and the upstream checksum."""
    g = golden("mse")
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(65536, 128, generator=gen)
    x /= x.norm(dim=-1, keepdim=True)
    rot = orc.make_rotation_matrix(128, 42)
    bnd, cent = orc.lloyd_max_codebook(4, 128)
    packed, norms = tq.quantize_mse(x.cuda(), 4, rotation=cuda(rot), codebook=(cuda(bnd), cuda(cent)))
    o_packed, o_norms, rotated = orc.quantize_mse(x.numpy(), 4, rot, bnd, return_rotated=True)
    rate, worst = code_mismatches(orc, packed.cpu().numpy(), o_packed, rotated, bnd, 4, 128)
    assert rate <= MAX_TIE_RATE, f"mismatch rate {rate:.2e}"
    np.testing.assert_allclose(norms.cpu().numpy(), o_norms, rtol=2e-6)
    diff = np.abs(packed.cpu().numpy().astype(np.int64).sum(0) - g["unit_packed_colsum"])
    assert diff.max() <= 256 and (diff > 0).sum() <= 16
    recon = tq.dequantize_mse(packed, norms, 4, 128, rotation=cuda(rot), codebook=(cuda(bnd), cuda(cent)))
    mse = float(((x.cuda() - recon) ** 2).sum(-1).mean())
    assert abs(mse - float(g["unit_mse_per_vector"])) < 1e-6


@pytest.mark.parametrize("n", [0, 1, 7, 8, 9, 63, 64, 65, 1000])
@pytest.mark.parametrize("dim", [8, 24, 64, 72, 128, 200, 256])
def test_quantize_mse_ragged_shapes(tq, orc, n, dim):
    rng = np.random.default_rng(n * 1000 + dim)
    x = rng.normal(size=(n, dim)).astype(np.float32)
    rot = orc.make_rotation_matrix(dim, 3)
    bnd, cent = orc.lloyd_max_codebook(3, dim)
    packed, norms = tq.quantize_mse(cuda(x), 3, rotation=cuda(rot), codebook=(cuda(bnd), cuda(cent)))
    assert packed.shape == (n, 3 * ((dim + 7) // 8)) and norms.shape == (n,)
    if n == 0:
        return
    o_packed, o_norms, rotated = orc.quantize_mse(x, 3, rot, bnd, return_rotated=True)
    code_mismatches(orc, packed.cpu().numpy(), o_packed, rotated, bnd, 3, dim)
    np.testing.assert_allclose(norms.cpu().numpy(), o_norms, rtol=2e-6)
    recon = tq.dequantize_mse(packed, norms, 3, dim, rotation=cuda(rot), codebook=(cuda(bnd), cuda(cent)))
    o_recon = orc.dequantize_mse(packed.cpu().numpy(), norms.cpu().numpy(), 3, dim, rot, cent)
    np.testing.assert_allclose(recon.cpu().numpy(), o_recon, rtol=1e-4, atol=1e-5 * max(np.abs(o_recon).max(), 1e-30))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_quantize_half_inputs_compute_in_float32(tq, orc, dtype):
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(513, 64, generator=gen).to(dtype)
    rot = orc.make_rotation_matrix(64, 42)
    bnd, cent = orc.lloyd_max_codebook(4, 64)
    packed, norms = tq.quantize_mse(x.cuda(), 4, rotation=cuda(rot), codebook=(cuda(bnd), cuda(cent)))
    o_packed, o_norms, rotated = orc.quantize_mse(x.float().numpy(), 4, rot, bnd, return_rotated=True)
    rate, _ = code_mismatches(orc, packed.cpu().numpy(), o_packed, rotated, bnd, 4, 64)
    assert rate <= 1e-3 and norms.dtype == torch.float32
    np.testing.assert_allclose(norms.cpu().numpy(), o_norms, rtol=2e-6)


@pytest.mark.parametrize("dim", [128, 64])
def test_quantize_prod_golden_and_oracle(tq, orc, golden, dim):
    g = golden("prod")
    x = g[f"x_d{dim}"]
    rot = orc.make_rotation_matrix(dim, 42)
    S = orc.make_qjl_matrix(dim, dim, 42)
    for bits in (2, 3, 4):
        bnd, cent = orc.lloyd_max_codebook(bits - 1, dim)
        mp, sg, rn, nm = tq.quantize_prod(cuda(x), bits, rotation=cuda(rot), codebook=(cuda(bnd), cuda(cent)),
                                          S_matrix=cuda(S))
        o_mp, o_sg, o_rn, o_nm, proj = orc.quantize_prod(x, bits, rot, bnd, cent, S, return_projected=True)
        a = orc.unpack_codes(mp.cpu().numpy(), bits - 1, dim)
        b = orc.unpack_codes(o_mp, bits - 1, dim)
        rows_ok = (a == b).all(axis=1)
        assert (~rows_ok).mean() <= 0.01
        sa = orc.unpack_codes(sg.cpu().numpy(), 1, dim)
        sb = orc.unpack_codes(o_sg, 1, dim)
        bad = np.argwhere((sa != sb) & rows_ok[:, None])
        scale = np.abs(proj).max()
        for r, j in bad:
            assert abs(proj[r, j]) < 1e-5 * scale, "sign differs away from a zero projection"
        assert len(bad) / sa.size <= 1e-3
        # and against the upstream package's own output
        gb = orc.unpack_codes(g[f"signs_b{bits}_d{dim}"], 1, dim)
        assert ((sa != gb) & rows_ok[:, None]).mean() <= 1e-3
        np.testing.assert_allclose(nm.cpu().numpy(), g[f"norms_b{bits}_d{dim}"], rtol=2e-6)
        np.testing.assert_allclose(rn.cpu().numpy()[rows_ok], o_rn[rows_ok], rtol=1e-4, atol=1e-6)
        recon = tq.dequantize_prod(cuda(g[f"mse_packed_b{bits}_d{dim}"]), cuda(g[f"signs_b{bits}_d{dim}"]),
                                   cuda(g[f"res_norms_b{bits}_d{dim}"]), cuda(g[f"norms_b{bits}_d{dim}"]), bits, dim,
                                   rotation=cuda(rot), codebook=(cuda(bnd), cuda(cent)), S_matrix=cuda(S))
        ref = g[f"recon_b{bits}_d{dim}"]
        np.testing.assert_allclose(recon.cpu().numpy()[:64], ref, rtol=1e-4, atol=1e-5 * np.abs(ref).max())


def test_prod_estimator_is_unbiased(tq, orc):
    """The Algorithm 2 property the upstream tests check: <q, dequantize_prod(x)> estimates <q, x> without bias."""
    gen = torch.Generator().manual_seed(1)
    sig = torch.exp(torch.empty(128).uniform_(np.log(0.1), np.log(10.0), generator=gen)).sqrt()
    x = torch.randn(20000, 128, generator=gen) * sig
    x /= x.norm(dim=-1, keepdim=True)
    q = torch.randn(64, 128, generator=gen) * sig
    q /= q.norm(dim=-1, keepdim=True)
    xs = x.cuda()
    mp, sg, rn, nm = tq.quantize_prod(xs, 3)
    recon = tq.dequantize_prod(mp, sg, rn, nm, 3, 128)
    exact = q.cuda() @ xs.t()
    est = q.cuda() @ recon.t()
    err = (est - exact).flatten()
    assert abs(float(err.mean())) < 4 * float(err.std()) / np.sqrt(err.numel()) + 1e-5
    slope = float((est * exact).sum() / (exact * exact).sum())
    assert abs(slope - 1.0) < 0.01


def test_errors_are_loud(tq):
    x = torch.randn(4, 64, device="cuda")
    with pytest.raises(ValueError):
        tq.quantize_prod(x, 1)
    with pytest.raises(RuntimeError):
        tq.quantize_mse(x, 5)
    with pytest.raises(RuntimeError):
        tq.quantize_mse(torch.randn(4, 260, device="cuda"), 4, rotation=torch.eye(260), codebook=tq.lloyd_max_codebook(4, 260))
    with pytest.raises(RuntimeError):
        tq.unpack_codes(torch.zeros(3, 5, dtype=torch.uint8, device="cuda"), 4, 64)
