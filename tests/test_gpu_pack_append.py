"""Quantise-on-append on the GPU against the oracle: bit-exact bytes and scales."""
import numpy as np
import pytest
import torch

from oracle import jf_oracle as O
from jf_testlib import to_bits, f32_values

pytestmark = pytest.mark.gpu
GOLD = np.load(__import__("pathlib").Path(__file__).parent / "golden" / "pack_golden.npz")


def _ops():
    from jetfire_b200 import ops
    return ops


@pytest.mark.parametrize("dt", ("bf16", "fp16"))
@pytest.mark.parametrize("bits", (2, 3, 4))
@pytest.mark.parametrize("gs", (64, 128))
def test_golden_rows_bit_exact(dt, bits, gs):
    """The committed outputs of the reference's quantize_and_pack, reproduced on the GPU."""
    ops = _ops()
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    x = torch.from_numpy(GOLD[f"x_{dt}"].view(np.int16).copy()).view(tdt)   # (R, 128)
    rows = x.shape[0]
    x_tok = x.reshape(rows, 1, 128).cuda()
    slots = torch.arange(rows, dtype=torch.int64, device="cuda")
    data = torch.zeros(1, rows, 16 * bits, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(1, rows, 128 // gs, dtype=torch.bfloat16, device="cuda")
    getattr(ops, f"fused_quant_write_int{bits}_sym")(x_tok, slots, data, scales, gs)
    torch.cuda.synchronize()
    key = f"{dt}_b{bits}_g{gs}"
    assert np.array_equal(to_bits(scales[0]), GOLD[key + "_scales"])
    assert np.array_equal(data[0].cpu().numpy(), GOLD[key + "_data"])


@pytest.mark.parametrize("bits,gs", [(3, 64), (2, 64), (4, 128), (4, 64), (2, 128), (3, 128)])
def test_scatter_permuted_slots_and_skip(bits, gs):
    """Permuted slots, a masked (-1) row, strided input, canary bytes untouched
    (the reference's write_cache check, scripts/validate_runtime.py:61-99)."""
    ops = _ops()
    g = torch.Generator().manual_seed(100 + bits + gs)
    T, H = 333, 3
    base = torch.randn(T + 1, H + 2, 128, generator=g).to(torch.bfloat16).cuda()
    x = base[:, 1:1 + H]                      # non-contiguous view: strides (5*128, 128, 1)
    slots = torch.randperm(T, generator=g).to(torch.int64)
    masked = torch.cat([slots, torch.tensor([-1])]).cuda()
    data = torch.full((H, T + 1, 16 * bits), 0xA5, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(H, T + 1, 128 // gs, dtype=torch.bfloat16, device="cuda")
    getattr(ops, f"fused_quant_write_int{bits}_sym")(x, masked, data, scales, gs)
    torch.cuda.synchronize()
    ref_d, ref_s = O.quantize_and_pack(f32_values(x[:T]), gs, bits)         # (T, H, Dp)
    got_d = data[:, slots.cuda()].transpose(0, 1).cpu().numpy()
    got_s = to_bits(scales[:, slots.cuda()].transpose(0, 1))
    assert np.array_equal(got_s, ref_s)
    assert np.array_equal(got_d, ref_d)
    assert bool((data[:, -1] == 0xA5).all()), "negative slot wrote to the cache"


@pytest.mark.parametrize("dt", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("bits,gs", [(3, 64), (2, 64), (4, 128)])
def test_rounding_boundaries_and_many_rows(dt, bits, gs):
    """Quotients that sit exactly on k + 1/2 (scale 1, 2^-3, 3: ties go to even), quotients one
    ulp either side of a boundary, and a large random batch, all bit-exact against the oracle."""
    ops = _ops()
    qmax = (1 << (bits - 1)) - 1
    g = torch.Generator().manual_seed(7 + bits)
    rows = []
    for scale in (1.0, 0.125, 3.0):
        halves = (torch.arange(128, dtype=torch.float32) % (2 * qmax + 2) - qmax - 0.5) * scale   # ..., -1.5, -0.5, 0.5, ...
        halves[::gs] = qmax * scale                                        # pins amax, hence the scale
        rows.append(halves)
        rows.append(-halves)
    x = torch.stack(rows)
    near = x.clone().to(dt)
    bump = torch.nextafter(near.float(), torch.full_like(near.float(), 1e9)).to(dt)
    x = torch.cat([x.to(dt), bump, torch.randn(4096, 128, generator=g).to(dt) * 3.0])
    n = x.shape[0]
    x_tok = x.reshape(n, 1, 128).cuda()
    slots = torch.arange(n, dtype=torch.int64, device="cuda")
    data = torch.zeros(1, n, 16 * bits, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(1, n, 128 // gs, dtype=torch.bfloat16, device="cuda")
    getattr(ops, f"fused_quant_write_int{bits}_sym")(x_tok, slots, data, scales, gs)
    torch.cuda.synchronize()
    ref_d, ref_s = O.quantize_and_pack(f32_values(x), gs, bits)
    assert np.array_equal(to_bits(scales[0]), ref_s)
    assert np.array_equal(data[0].cpu().numpy(), ref_d)


def test_kv_pair_and_out_of_range_slot():
    ops = _ops()
    g = torch.Generator().manual_seed(7)
    T, H = 40, 2
    k = torch.randn(T, H, 128, generator=g).to(torch.float16).cuda()
    v = torch.randn(T, H, 128, generator=g).to(torch.float16).cuda()
    slots = torch.arange(T, dtype=torch.int64)
    slots[5] = 10_000            # beyond num_slots: must be skipped, not written
    slots = slots.cuda()
    kd = torch.full((H, 64, 48), 0xA5, dtype=torch.uint8, device="cuda")
    vd = torch.full((H, 64, 32), 0xA5, dtype=torch.uint8, device="cuda")
    ks = torch.zeros(H, 64, 2, dtype=torch.bfloat16, device="cuda")
    vs = torch.zeros_like(ks)
    ops.fused_quant_write_kv(k, v, slots, kd, ks, vd, vs, 64, 3, 2)
    torch.cuda.synchronize()
    rk, rks = O.quantize_and_pack(f32_values(k), 64, 3)
    rv, rvs = O.quantize_and_pack(f32_values(v), 64, 2)
    keep = [t for t in range(T) if t != 5]
    assert np.array_equal(kd[:, keep].transpose(0, 1).cpu().numpy(), rk[keep])
    assert np.array_equal(vd[:, keep].transpose(0, 1).cpu().numpy(), rv[keep])
    assert np.array_equal(to_bits(ks[:, keep].transpose(0, 1)), rks[keep])
    assert np.array_equal(to_bits(vs[:, keep].transpose(0, 1)), rvs[keep])
    assert bool((kd[:, 5] == 0xA5).all()) and bool((kd[:, T:] == 0xA5).all())


def test_rejects_bad_arguments():
    ops = _ops()
    x = torch.zeros(4, 2, 128, dtype=torch.float32, device="cuda")
    slots = torch.arange(4, dtype=torch.int64, device="cuda")
    data = torch.zeros(2, 16, 48, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(2, 16, 2, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        ops.fused_quant_write_int3_sym(x, slots, data, sc, 64)          # fp32 input
    with pytest.raises(RuntimeError):
        ops.fused_quant_write_int3_sym(x.bfloat16(), slots, data, sc, 32)  # bad group
