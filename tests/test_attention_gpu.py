"""tcgen05 flash-attention kernels against a plain fp32 PyTorch restatement (forward output,
log-sum-exp, and the gradient with respect to the packed projection), MHA and GQA."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(qkv, rep, dout):
    """fp32 attention over the packed group-major layout with autograd for the gradient."""
    x = qkv.float().detach().requires_grad_(True)
    B, S, H, D = x.shape
    hkv = H // (rep + 2)
    g = x.view(B, S, hkv, rep + 2, D)
    q = g[:, :, :, :rep].reshape(B, S, hkv * rep, D).permute(0, 2, 1, 3)
    k = g[:, :, :, rep].permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    v = g[:, :, :, rep + 1].permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = q @ k.transpose(-1, -2) / math.sqrt(D)
    mask = torch.ones(S, S, dtype=torch.bool, device=x.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = (torch.softmax(s, dim=-1) @ v).permute(0, 2, 1, 3)
    (dx,) = torch.autograd.grad(o, x, dout.float())
    return o.detach(), lse.detach(), dx


@pytest.mark.parametrize("B,S,hkv,rep", [(2, 256, 2, 1), (1, 512, 2, 4), (1, 1024, 1, 2), (2, 128, 3, 1)])
def test_flash_attention_matches_fp32_reference(B, S, hkv, rep):
    from multimesh_jax_b200.ops import attention, kernels as K
    torch.manual_seed(S + rep)
    dev = torch.device("cuda")
    D = 128
    qkv = (torch.randn(B, S, hkv * (rep + 2), D, device=dev) * 0.7).bfloat16()
    dout = torch.randn(B, S, hkv * rep, D, device=dev).bfloat16()
    assert attention.native_supported(qkv)
    before = K.library_call_count
    out, lse = attention.attention_fwd_packed(qkv, rep)
    dqkv = attention.attention_bwd_packed(dout, qkv, out, lse, rep)
    torch.cuda.synchronize()
    assert K.library_call_count == before          # no library attention on this path
    assert K.read_status() == 0
    o_ref, lse_ref, dx_ref = _reference(qkv, rep, dout)
    torch.testing.assert_close(out.float(), o_ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, lse_ref, rtol=1e-3, atol=2e-3)
    err = (dqkv.float() - dx_ref).abs().max().item() / dx_ref.abs().max().item()
    assert err < 2e-2, err
    # relative Frobenius errors: probabilities and dS are rounded to bf16 before their products
    fro = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert fro(out, o_ref) < 1e-2, fro(out, o_ref)
    # per-slot check so that a wrong key or value gradient cannot hide behind the query's
    g = dqkv.float().view(B, S, hkv, rep + 2, D)
    gr = dx_ref.view(B, S, hkv, rep + 2, D)
    for slot in (0, rep, rep + 1):
        e = (g[:, :, :, slot] - gr[:, :, :, slot]).abs().max().item() / gr[:, :, :, slot].abs().max().item()
        assert e < 3e-2, (slot, e)
        assert fro(g[:, :, :, slot], gr[:, :, :, slot]) < 2e-2, (slot, fro(g[:, :, :, slot], gr[:, :, :, slot]))


def test_flash_attention_twice_in_a_row_is_deterministic_in_forward():
    from multimesh_jax_b200.ops import attention
    dev = torch.device("cuda")
    qkv = torch.randn(1, 256, 6, 128, device=dev).bfloat16()
    a, la = attention.attention_fwd_packed(qkv, 1)
    b, lb = attention.attention_fwd_packed(qkv, 1)
    assert torch.equal(a, b) and torch.equal(la, lb)
