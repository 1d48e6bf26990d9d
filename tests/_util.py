"""Shared helpers for the parity tests."""
import torch

# Tolerances of the bf16 CUDA path against the fp32 oracle evaluated on the same bf16-rounded
# inputs: max-abs <= 2e-2 and mean-abs <= 2e-3 on outputs and gradients; selected block indices
# bit-exact except where the competing scores are within 1e-3.
MAX_ABS = 2e-2
MEAN_ABS = 2e-3
TIE_EPS = 1e-3


def assert_bf16_close(got: torch.Tensor, ref: torch.Tensor, what: str = "", max_abs: float = MAX_ABS,
                      mean_abs: float = MEAN_ABS, scale_with_ref: bool = True):
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values in the CUDA result"
    err = (got - ref).abs()
    # gradients can be large in magnitude; the tolerance is relative to the reference's scale when > 1
    s = max(1.0, ref.abs().max().item()) if scale_with_ref else 1.0
    assert err.max().item() <= max_abs * s, f"{what}: max-abs {err.max().item():.4g} > {max_abs * s:.4g}"
    assert err.mean().item() <= mean_abs * s, f"{what}: mean-abs {err.mean().item():.4g} > {mean_abs * s:.4g}"


def assert_idx_match(idx_gpu: torch.Tensor, idx_ref: torch.Tensor, scores: torch.Tensor, what: str = "",
                     eps: float = TIE_EPS, exact: bool = False):
    """idx_* [...,Nq,K] int32; scores [...,Nq,Nc] fp32 raw logits of the oracle.  Entries must be
    identical, except that where they differ the two selected scores must be within ``eps``."""
    a, b = idx_gpu.cpu().long(), idx_ref.cpu().long()
    assert a.shape == b.shape, f"{what}: idx shape {tuple(a.shape)} vs {tuple(b.shape)}"
    Nc = scores.shape[-1]
    assert (a >= 0).all() and (a < Nc).all(), f"{what}: index out of range"
    diff = a != b
    if exact:
        assert not diff.any(), f"{what}: {int(diff.sum())} index entries differ (exact match required)"
        return 0
    if diff.any():
        sa = torch.gather(scores, -1, a)
        sb = torch.gather(scores, -1, b)
        bad = diff & ((sa - sb).abs() > eps)
        assert not bad.any(), (f"{what}: {int(bad.sum())} index entries differ beyond a {eps} tie "
                               f"(max score gap {((sa - sb).abs() * diff).max().item():.4g})")
    return int(diff.sum())


def bf16_round(*ts):
    return [t.to(torch.bfloat16).float() for t in ts]


# ------------------------------------------------------------------------------------------------
# device-side cross-checks: the tests-only companion library (include/speed3r_b200_check.h)
# ------------------------------------------------------------------------------------------------
def _check_call(rc, what):
    import ctypes as C
    from speed3r_b200 import _lib
    if rc != 0:
        buf = C.create_string_buffer(512)
        _lib.load_check().s3r_last_error(buf, 512)
        raise RuntimeError(f"{what} failed with code {rc}: {buf.value.decode(errors='replace')}")


def check_cmp_attn_topk(q_c, k_c, v_c, topk, scale=None):
    import math
    from speed3r_b200 import _lib
    B, H, Nq, d = q_c.shape
    Nc = k_c.shape[2]
    scale = scale or 1.0 / math.sqrt(d)
    o = torch.empty_like(q_c)
    lse = torch.empty(B, H, Nq, device=q_c.device, dtype=torch.float32)
    idx = torch.empty(B, H, Nq, topk, device=q_c.device, dtype=torch.int32)
    _check_call(_lib.load_check().s3r_check_cmp_attn_topk_fwd(
        q_c.data_ptr(), k_c.data_ptr(), v_c.data_ptr(), o.data_ptr(), lse.data_ptr(), idx.data_ptr(), B, H, Nq, Nc, d,
        topk, scale, torch.cuda.current_stream().cuda_stream), "s3r_check_cmp_attn_topk_fwd")
    return o, lse, idx


def check_sel_attn(q, k, v, idx, block, scale=None):
    import math
    from speed3r_b200 import _lib
    B, H, Tq, d = q.shape
    Tk = k.shape[2]
    scale = scale or 1.0 / math.sqrt(d)
    o = torch.empty_like(q)
    lse = torch.empty(B, H, Tq, device=q.device, dtype=torch.float32)
    _check_call(_lib.load_check().s3r_check_sel_attn_fwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), idx.data_ptr(), o.data_ptr(), lse.data_ptr(), B, H, Tq, Tk, d, block,
        idx.shape[-1], scale, torch.cuda.current_stream().cuda_stream), "s3r_check_sel_attn_fwd")
    return o, lse
