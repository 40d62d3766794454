"""fa_rotary_qkv (one pass over a packed qkv tensor) against the formulation of the reference
(flash_attn/rotary.py:33-43: x * cos + rotate_half(x) * sin on q and k, v untouched)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(qkv):
    """The reference's arithmetic in fp32: pairs (2i, 2i+1) rotated by pos * 10000^(-2i/d)."""
    b, s, _, h, d = qkv.shape
    inv_freq = 1.0 / (10000 ** (torch.arange(0, d, 2, device=qkv.device).float() / d))
    ang = torch.outer(torch.arange(s, device=qkv.device).float(), inv_freq)       # (s, d/2)
    cos = torch.cos(ang).repeat_interleave(2, dim=-1)[None, :, None, :]
    sin = torch.sin(ang).repeat_interleave(2, dim=-1)[None, :, None, :]

    def rot(x):
        x = x.float()
        x1, x2 = x[..., 0::2], x[..., 1::2]
        half = torch.stack((-x2, x1), dim=-1).flatten(-2)
        return x * cos + half * sin

    return torch.stack([rot(qkv[:, :, 0]), rot(qkv[:, :, 1]), qkv[:, :, 2].float()], dim=2)


@pytest.mark.parametrize("dtype,b,s,h,d", [(torch.float16, 2, 37, 3, 64), (torch.bfloat16, 3, 128, 2, 128),
                                           (torch.float16, 1, 5, 1, 16), (torch.bfloat16, 2, 300, 4, 32)])
def test_rotary_qkv_matches_reference_formula(dtype, b, s, h, d):
    from flash_attn_b200.rotary import RotaryEmbedding
    g = torch.Generator(device="cuda").manual_seed(b * s + d)
    qkv = torch.randn(b, s, 3, h, d, device="cuda", generator=g).to(dtype)
    rope = RotaryEmbedding(d).cuda()
    assert rope.fused_path(qkv)
    got = rope.apply_qkv(qkv)
    want = _reference(qkv)
    # one rounding to the 16-bit type on top of fp32 arithmetic
    eps = 2.0 ** -8 if dtype is torch.bfloat16 else 2.0 ** -11
    assert (got.float() - want).abs().max().item() <= eps * want.abs().max().item() + 1e-6
    assert torch.equal(got[:, :, 2], qkv[:, :, 2])                     # v is a plain copy
    # and it equals the module's own unfused path to the last bit or one unit in the last place
    q, k = rope(qkv[:, :, 0], qkv[:, :, 1], seq_dimension=-3)
    assert (got[:, :, 0].float() - q.float()).abs().max().item() <= eps * want.abs().max().item()
    assert (got[:, :, 1].float() - k.float()).abs().max().item() <= eps * want.abs().max().item()


def test_rotary_qkv_gradient_is_the_inverse_rotation():
    from flash_attn_b200.rotary import RotaryEmbedding
    b, s, h, d = 2, 50, 2, 64
    qkv = torch.randn(b, s, 3, h, d, device="cuda", dtype=torch.float16, requires_grad=True)
    rope = RotaryEmbedding(d).cuda()
    out = rope.apply_qkv(qkv)
    w = torch.randn_like(out)
    (out.float() * w.float()).sum().backward()
    ref_in = qkv.detach().float().requires_grad_()
    (_reference(ref_in) * w.float()).sum().backward()
    assert (qkv.grad.float() - ref_in.grad).abs().max().item() <= 2.0 ** -10 * ref_in.grad.abs().max().item()
    # a rotation preserves the norm of every (q or k) head vector
    assert torch.allclose(out[:, :, :2].float().norm(dim=-1), qkv[:, :, :2].detach().float().norm(dim=-1),
                          rtol=2e-3, atol=1e-3)


def test_flash_mha_uses_the_fused_rotation():
    from flash_attn_b200.flash_attention import FlashMHA
    torch.manual_seed(0)
    mha = FlashMHA(128, 2, use_rotary_emb="1d", device="cuda", dtype=torch.float16)
    x = torch.randn(2, 64, 128, device="cuda", dtype=torch.float16)
    y, _ = mha(x)
    # unfused route through the same module
    qkv = mha.Wqkv(x).reshape(2, 64, 3, 2, 64)
    q, k, v = qkv.unbind(dim=2)
    q, k = mha.rotary_emb(q, k, seq_dimension=-3)
    ctx, _ = mha.inner_attn(torch.stack([q, k, v], dim=2), causal=False)
    y2 = mha.out_proj(ctx.reshape(2, 64, 128))
    assert (y.float() - y2.float()).abs().max().item() < 5e-3


@pytest.mark.parametrize("dtype,b,side,h,d", [(torch.float16, 2, 7, 3, 64), (torch.bfloat16, 1, 16, 2, 128),
                                              (torch.float16, 2, 5, 1, 32)])
def test_rotary_2d_qkv_matches_the_unfused_module(dtype, b, side, h, d):
    """The 2-D embedding through the one-pass kernel (a per-position table of column / row angles)
    against the module's framework-op path, which follows flash_attn/rotary.py:103-135."""
    from flash_attn_b200.rotary import RotaryEmbedding2D
    s = side * side
    g = torch.Generator(device="cuda").manual_seed(side + d)
    qkv = torch.randn(b, s, 3, h, d, device="cuda", generator=g).to(dtype)
    rope = RotaryEmbedding2D(d).cuda()
    got = rope.apply_qkv(qkv)
    q, k = rope(qkv[:, :, 0].float(), qkv[:, :, 1].float(), seq_dimension=-3)
    eps = 2.0 ** -8 if dtype is torch.bfloat16 else 2.0 ** -11
    scale = max(q.abs().max().item(), k.abs().max().item())
    assert (got[:, :, 0].float() - q).abs().max().item() <= eps * scale + 1e-6
    assert (got[:, :, 1].float() - k).abs().max().item() <= eps * scale + 1e-6
    assert torch.equal(got[:, :, 2], qkv[:, :, 2])
    # token 0 (row 0, column 0) is not rotated at all; token 1 (column 1) only in its first half
    assert torch.equal(got[:, 0, :2], qkv[:, 0, :2])
    assert torch.equal(got[:, 1, :2, :, d // 2:], qkv[:, 1, :2, :, d // 2:])


def test_flash_mha_2d_rotary_runs_fused():
    from flash_attn_b200.flash_attention import FlashMHA
    torch.manual_seed(0)
    mha = FlashMHA(128, 2, use_rotary_emb="2d", device="cuda", dtype=torch.float16)
    x = torch.randn(2, 49, 128, device="cuda", dtype=torch.float16)
    y, _ = mha(x)
    qkv = mha.Wqkv(x).reshape(2, 49, 3, 2, 64)
    q, k, v = qkv.unbind(dim=2)
    q, k = mha.rotary_emb(q, k, seq_dimension=-3)
    ctx, _ = mha.inner_attn(torch.stack([q, k, v], dim=2), causal=False)
    y2 = mha.out_proj(ctx.reshape(2, 49, 128))
    assert (y.float() - y2.float()).abs().max().item() < 5e-3
