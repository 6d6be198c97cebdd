"""Weight layout helpers (host side, one-off at load time).

The reference's RDNA kernels take B pre-shuffled for the WMMA operand layout,
``dst[n0, k0, kl, l16, kp] = B[k0*16 + kl*8 + kp, n0*16 + l16]`` with shape ``[N/16, K/16, 2, 16, 8]``
(``preshuffle_b_fp8`` fly/rdna_fp8_preshuffle_gemm.py:40-54, ``preshuffle_b_f16``
fly/rdna_fp8_factored_gemm.py:56-61).  The B200 kernels read weights K-major ``[N, K]`` through TMA, so callers
that hold the RDNA layout convert once with the functions below; ``preshuffle_b`` is the forward mapping."""
import torch


def preshuffle_b(B_kn):
    """``B[K, N]`` (any 1- or 2-byte dtype) -> ``[N/16, K/16, 2, 16, 8]`` as the reference lays it out."""
    K, N = B_kn.shape
    if K % 16 or N % 16:
        raise ValueError("K and N must be multiples of 16")
    v = B_kn.view(torch.uint8) if B_kn.element_size() == 1 else B_kn
    return v.reshape(K // 16, 2, 8, N // 16, 16).permute(3, 0, 1, 4, 2).contiguous()


def unshuffle_b(B_shuf):
    """Inverse of :func:`preshuffle_b`, returning the K-major weight ``W[N, K] = B^T`` the B200 library takes."""
    n0, k0, kl, l16, kp = B_shuf.shape
    if (kl, l16, kp) != (2, 16, 8):
        raise ValueError("expected [N/16, K/16, 2, 16, 8]")
    return B_shuf.permute(0, 3, 1, 2, 4).reshape(n0 * 16, k0 * 16).contiguous()


def unshuffle_b_fp8(B_shuf_u8):
    """Pre-shuffled E4M3 bytes -> ``float8_e4m3fn`` ``[N, K]``."""
    return unshuffle_b(B_shuf_u8).view(torch.float8_e4m3fn)


def split_fc1(fc1_kn, N):
    """``fc1[K, 2N]`` -> (gate ``[N, K]``, up ``[N, K]``): gate = first N columns, up = last N
    (``split_and_preshuffle_fc1``, fly/rdna_fp8_dual_gemm_silu.py:53-63), K-major for this library."""
    return fc1_kn[:, :N].t().contiguous(), fc1_kn[:, N:2 * N].t().contiguous()
