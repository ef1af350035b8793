"""EnhancedMultiHeadAttention: mask handling on the CPU, the layer against plain PyTorch on the GPU."""
import pytest
import torch
import torch.nn.functional as F

import flash_attention_v100 as fa
from flash_attention_v100.modules import masks_to_bias
from flash_attention_v100.testing import rel_l2


def test_masks_become_the_smallest_bias():
    B, Nq, Nk = 2, 5, 7
    pad = torch.zeros(B, Nk, dtype=torch.bool)
    pad[:, 5:] = True
    b = masks_to_bias(None, pad, B, Nq, Nk)
    assert b.shape == (B, 1, 1, Nk) and b.dtype == torch.float32
    assert torch.isinf(b[..., 5:]).all() and (b[..., :5] == 0).all()
    am = torch.triu(torch.ones(Nq, Nk, dtype=torch.bool), diagonal=1)
    b2 = masks_to_bias(am, None, B, Nq, Nk)
    assert b2.shape == (1, 1, Nq, Nk)
    b3 = masks_to_bias(am, pad, B, Nq, Nk)
    assert b3.shape == (B, 1, Nq, Nk)
    assert torch.equal(torch.isinf(b3), (am.view(1, 1, Nq, Nk) | pad.view(B, 1, 1, Nk)))
    fm = torch.randn(B, Nq, Nk)
    assert torch.equal(masks_to_bias(fm, None, B, Nq, Nk), fm.view(B, 1, Nq, Nk))
    assert masks_to_bias(None, None, B, Nq, Nk) is None
    with pytest.raises(ValueError):
        masks_to_bias(torch.zeros(3, 3), None, B, Nq, Nk)
    with pytest.raises(ValueError):
        masks_to_bias(None, torch.zeros(B, Nk + 1), B, Nq, Nk)


def test_compact_keys_moves_the_kept_keys_to_the_front():
    from flash_attention_v100.modules import compact_keys
    torch.manual_seed(1)
    B, Nk, H, D = 3, 9, 2, 4
    k, v = torch.randn(B, Nk, H, D), torch.randn(B, Nk, H, D)
    pad = torch.zeros(B, Nk, dtype=torch.bool)
    pad[0, [1, 4, 8]] = True            # holes
    pad[1, :] = True                    # everything hidden
    k2, v2, counts = compact_keys(k, v, pad)
    assert counts.dtype == torch.int32 and counts.tolist() == [6, 1, 9]
    assert torch.equal(k2[0, :6], k[0, [0, 2, 3, 5, 6, 7]]) and torch.equal(v2[0, :6], v[0, [0, 2, 3, 5, 6, 7]])
    assert torch.equal(k2[2], k[2])
    # attention over the first counts[b] keys of the compacted tensors = masked attention over the originals
    q = torch.randn(B, 5, H, D)
    for b in (0, 2):
        s_full = torch.einsum("ihd,jhd->hij", q[b], k[b]).masked_fill(pad[b].view(1, 1, Nk), float("-inf"))
        o_full = torch.einsum("hij,jhd->ihd", s_full.softmax(-1), v[b])
        n = int(counts[b])
        s_c = torch.einsum("ihd,jhd->hij", q[b], k2[b, :n])
        o_c = torch.einsum("hij,jhd->ihd", s_c.softmax(-1), v2[b, :n])
        assert torch.allclose(o_full, o_c, atol=1e-6)
    with pytest.raises(ValueError):
        compact_keys(k, v, pad.float())


def test_a_boolean_key_padding_mask_alone_reaches_the_kernels_as_key_counts(monkeypatch):
    import flash_attention_v100.modules as m
    seen = {}

    def spy(q, k, v, **kw):
        seen.update(kw)
        return torch.zeros_like(q)

    monkeypatch.setattr(m, "flash_attention_v100", spy)
    layer = fa.EnhancedMultiHeadAttention(32, 2, enable_multi_gpu=False)
    x = torch.randn(2, 6, 32)
    pad = torch.zeros(2, 6, dtype=torch.bool)
    pad[0, 2] = True
    layer(x, key_padding_mask=pad)
    assert seen["bias"] is None and seen["key_lengths"].tolist() == [5, 6]
    layer(x, key_padding_mask=pad, is_causal=True)                     # the causal mask depends on positions
    assert seen["bias"] is not None and seen["key_lengths"] is None
    layer(x, key_padding_mask=pad.float() * -1e4)                      # an additive mask stays a bias
    assert seen["bias"] is not None and seen["key_lengths"] is None


def test_layer_has_the_reference_parameter_names():
    layer = fa.EnhancedMultiHeadAttention(64, 4, bias=True)
    names = set(dict(layer.named_parameters()))
    assert names == {f"{p}_proj.{w}" for p in ("q", "k", "v", "out") for w in ("weight", "bias")}
    assert layer.head_dim == 16 and layer.get_performance_stats() is None
    with pytest.raises(ValueError):
        fa.EnhancedMultiHeadAttention(65, 4)


def _torch_reference(layer, x, key_padding_mask, attn_mask, is_causal):
    B, N, E = x.shape
    H, D = layer.num_heads, layer.head_dim
    q, k, v = (p(x).view(B, N, H, D).transpose(1, 2).float() for p in (layer.q_proj, layer.k_proj, layer.v_proj))
    mask = torch.zeros(B, 1, N, N, device=x.device)
    if key_padding_mask is not None:
        mask = mask.masked_fill(key_padding_mask.view(B, 1, 1, N), float("-inf"))
    if attn_mask is not None:
        mask = mask.masked_fill(attn_mask.view(1, 1, N, N), float("-inf"))
    if is_causal:
        mask = mask.masked_fill(torch.triu(torch.ones(N, N, dtype=torch.bool, device=x.device), 1), float("-inf"))
    o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
    return layer.out_proj(o.transpose(1, 2).reshape(B, N, E).to(x.dtype))


@pytest.mark.gpu
@pytest.mark.parametrize("masks", ["none", "padding", "padding+attn"])
def test_layer_matches_plain_pytorch(masks):
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    B, N, E, H = 2, 200, 256, 4
    layer = fa.EnhancedMultiHeadAttention(E, H, enable_multi_gpu=False).to(dev).to(torch.bfloat16).eval()
    x = (torch.randn(B, N, E, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    pad = attn = None
    if masks != "none":
        pad = torch.zeros(B, N, dtype=torch.bool, device=dev)
        pad[0, 150:] = True
        pad[1, 3::5] = True             # holes, not only a padded tail
    if masks == "padding+attn":
        attn = torch.zeros(N, N, dtype=torch.bool, device=dev)
        attn[:, ::7] = True
        attn.fill_diagonal_(False)
    out, weights = layer(x, key_padding_mask=pad, attn_mask=attn, is_causal=(masks == "none"))
    assert weights is None and out.shape == (B, N, E)
    ref = _torch_reference(layer, x, pad, attn, masks == "none")
    assert rel_l2(out, ref) < 1e-2
    out.float().square().sum().backward()
    assert torch.isfinite(x.grad).all() and torch.isfinite(layer.q_proj.weight.grad).all()
    # the gradients too, against autograd through the plain PyTorch layer (hidden keys get none)
    got = [x.grad.clone(), layer.k_proj.weight.grad.clone(), layer.v_proj.weight.grad.clone()]
    x.grad = None
    layer.zero_grad()
    ref.float().square().sum().backward()
    for g, r in zip(got, (x.grad, layer.k_proj.weight.grad, layer.v_proj.weight.grad)):
        assert rel_l2(g, r) < 3e-2
    x.grad = None
    layer.zero_grad()
    # sequence-first input gives the same result
    layer.batch_first = False
    out_sf, _ = layer(x.detach().transpose(0, 1), key_padding_mask=pad, attn_mask=attn, is_causal=(masks == "none"))
    assert torch.equal(out_sf.transpose(0, 1), out.detach())
