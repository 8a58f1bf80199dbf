"""Helpers of the full-size GPU parity tests: seeded sources drawn on the GPU (the host generator needs minutes
for 10^9 values), quantised by the library's own GPU quantisers (held byte-exact to the oracle by
tests/test_quantize_gpu.py), and oracle-side dequantisation of rows read back from the device."""
import numpy as np

from oracle import gemm_oracle as O


def draw(torch, shape, seed, dist="normal", scale=1.0):
    """Seeded fp32 tensor on the current GPU (Philox; the same values on every B200 for a given seed)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dist == "normal":
        return torch.randn(shape, generator=g, dtype=torch.float32, device="cuda") * scale
    return (torch.rand(shape, generator=g, dtype=torch.float32, device="cuda") * 2 - 1) * scale


def nvfp4_rows_from_device(torch, q_packed, sf_chunks, g, rows, k):
    """Dequantised fp32 values (oracle arithmetic) of the given rows of an NVFP4 operand that lives on the GPU:
    q_packed [R, K/2] bytes, sf_chunks the chunked scale table, g the per-tensor scale."""
    rows = np.asarray(rows)
    codes = O.unpack_e2m1(q_packed[torch.as_tensor(rows, device=q_packed.device)].cpu().numpy())
    kg = k // 64
    ch = sf_chunks.view(-1, kg, 512)
    rb, rr = rows // 128, rows % 128
    blocks = ch[torch.as_tensor(rb, device=ch.device)].cpu().numpy()            # [len(rows), kg, 512]
    off = (rr % 32) * 16 + (rr // 32) * 4
    s_bits = np.stack([blocks[i, :, off[i]:off[i] + 4].reshape(-1) for i in range(len(rows))])   # [len(rows), K/16]
    return O.dequantize_nvfp4(codes, s_bits, g)


def nvfp4_all_from_device(torch, q_packed, sf_chunks, g, n_rows, k, chunk=4096):
    """Generator of (first_row, dequantised rows) over the whole operand, `chunk` rows at a time."""
    for r0 in range(0, n_rows, chunk):
        rows = np.arange(r0, min(n_rows, r0 + chunk))
        yield r0, nvfp4_rows_from_device(torch, q_packed, sf_chunks, g, rows, k)
