"""Padded <-> packed copies, depthwise causal convolution over packed sequences, router: PyTorch paths on CPU, the
sm_100a kernels against them on a GPU."""

import pytest
import torch
import torch.nn.functional as F

from lm_engine.ops.sequence import (causal_conv1d_packed, compute_cu_seqlens_and_max_seqlen_from_attention_mask, pack_sequence,
                                    topk_route, unpack_sequence)


def _mask(lengths, seq, left, device):
    pos = torch.arange(seq, device=device).unsqueeze(0)
    lengths = torch.tensor(lengths, device=device).unsqueeze(1)
    return (pos >= seq - lengths) if left else (pos < lengths)


def _check_pack(device, dtype):
    lengths, seq = [5, 12, 1, 9], 12
    for left in (True, False):
        mask = _mask(lengths, seq, left, device)
        cu, max_len = compute_cu_seqlens_and_max_seqlen_from_attention_mask(mask.int())
        assert max_len == 12 and cu.tolist() == [0, 5, 17, 18, 27]
        x = torch.randn(4, seq, 3, 8, device=device).to(dtype).requires_grad_(True)
        side = "left" if left else "right"
        packed = pack_sequence(x, cu, side)
        assert packed.shape == (27, 3, 8) and torch.equal(packed, x[mask])
        back = unpack_sequence(packed, cu, (4, seq, 3, 8), side)
        assert torch.equal(back, x * mask[..., None, None].to(dtype))
        back.sum().backward()
        assert torch.equal(x.grad, mask[..., None, None].to(dtype).expand_as(x))


def _conv_reference(x, w, b, bounds, silu):
    k = w.shape[-1]
    out = []
    for s, e in zip(bounds[:-1], bounds[1:]):
        seq = F.pad(x[s:e].t().unsqueeze(0), (k - 1, 0))
        out.append(F.conv1d(seq, w.view(-1, 1, k), b, groups=x.shape[1]).squeeze(0).t())
    y = torch.cat(out)
    return F.silu(y) if silu else y


def _check_conv(device, dtype, tol):
    torch.manual_seed(0)
    bounds = [0, 7, 8, 40, 64]
    cu = torch.tensor(bounds, dtype=torch.int32, device=device)
    for k, silu, bias in ((4, True, True), (3, False, False), (1, True, True)):
        x = torch.randn(64, 48, device=device).to(dtype).requires_grad_(True)
        w = (torch.randn(48, 1, k, device=device) * 0.5).requires_grad_(True)
        b = torch.randn(48, device=device).requires_grad_(True) if bias else None
        y = causal_conv1d_packed(x, w, b, cu, "silu" if silu else None)
        xr, wr = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True)
        br = b.detach().clone().requires_grad_(True) if bias else None
        ref = _conv_reference(xr, wr, br, bounds, silu)
        torch.testing.assert_close(y.float(), ref, atol=tol, rtol=tol)
        dy = torch.randn_like(ref)
        y.backward(dy.to(dtype))
        ref.backward(dy)
        torch.testing.assert_close(x.grad.float(), xr.grad, atol=tol, rtol=tol)
        torch.testing.assert_close(w.grad, wr.grad, atol=10 * tol, rtol=tol)
        if bias:
            torch.testing.assert_close(b.grad, br.grad, atol=10 * tol, rtol=tol)


def _check_route(device, dtype):
    torch.manual_seed(1)
    for experts, k in ((8, 2), (40, 8), (64, 1), (200, 4)):
        logits = torch.randn(333, experts, device=device).to(dtype).requires_grad_(True)
        weights, chosen, counts = topk_route(logits, k, want_counts=True)
        ref_logits = logits.detach().float().requires_grad_(True)
        top, ref_chosen = ref_logits.topk(k, dim=-1)
        ref_weights = F.softmax(top, dim=-1)
        # equal logits (frequent in bf16) may be picked in another order: compare the selected values, not the indices
        assert torch.equal(ref_logits.detach().gather(1, chosen), top.detach())
        assert all(len(set(row)) == k for row in chosen[:50].tolist())
        torch.testing.assert_close(weights, ref_weights, atol=1e-5, rtol=1e-5)
        assert torch.equal(counts.long(), torch.bincount(chosen.flatten(), minlength=experts))
        dw = torch.randn_like(ref_weights)
        weights.backward(dw)
        ref_weights.backward(dw)
        mine = logits.grad.float().gather(1, chosen)
        theirs = ref_logits.grad.gather(1, ref_chosen)
        torch.testing.assert_close(mine, theirs, atol=2e-2 if dtype == torch.bfloat16 else 1e-5, rtol=1e-2)


def test_pack_unpack_cpu():
    _check_pack(torch.device("cpu"), torch.float32)


def test_causal_conv_cpu():
    _check_conv(torch.device("cpu"), torch.float32, 1e-5)


def test_route_cpu():
    _check_route(torch.device("cpu"), torch.float32)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_pack_unpack_gpu(dtype):
    _check_pack(torch.device("cuda"), dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 5e-2)])
def test_causal_conv_gpu(dtype, tol):
    _check_conv(torch.device("cuda"), dtype, tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_route_gpu(dtype):
    _check_route(torch.device("cuda"), dtype)
