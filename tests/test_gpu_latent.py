"""Latent <-> token layout kernels and the streaming hand-off of finished chunks (bit-exact: pure data movement)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_unpatchify_reference_order(u, C, f, h, w):
    """The reference's unpatchify (features (kh, kw, c))."""
    return torch.einsum("fhwpqrc->cfphqwr", u.view(f, h, w, 1, 2, 2, C)).reshape(C, f, 2 * h, 2 * w)


def _ref_patchify(lat):
    C, f, H, W = lat.shape
    h, w = H // 2, W // 2
    return lat.view(C, f, h, 2, w, 2).permute(1, 2, 4, 0, 3, 5).reshape(f * h * w, 4 * C)


@pytest.mark.parametrize("C,f,h,w", [(48, 3, 22, 40), (4, 3, 4, 6), (5, 1, 1, 1), (16, 2, 7, 33)])
def test_patchify_unpatchify(C, f, h, w):
    from longlive_b200 import checkpoint as ck
    from longlive_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(C + h)
    lat = torch.randn(C, f, 2 * h, 2 * w, device="cuda", generator=g).bfloat16()
    tok = ops.patchify(lat)
    assert torch.equal(tok, _ref_patchify(lat))
    back = torch.zeros_like(lat)
    assert torch.equal(ops.unpatchify(tok, back), lat)
    # [F, C, H, W] latents (the pipeline's layout) through strides
    lat_fc = lat.permute(1, 0, 2, 3).contiguous()
    assert torch.equal(ops.patchify(lat_fc, channels_first=False), tok)
    out_fc = torch.zeros_like(lat_fc)
    assert torch.equal(ops.unpatchify(tok, out_fc, channels_first=False), lat_fc)
    # a head in the reference's row order followed by the reference's unpatchify == permuted rows + this unpatchify
    u = torch.randn(f * h * w, 4 * C, device="cuda", generator=g).bfloat16()
    want = _ref_unpatchify_reference_order(u, C, f, h, w)
    got = ops.unpatchify(u[:, ck.head_row_order(C).cuda()].contiguous(), torch.empty_like(lat))
    assert torch.equal(got, want)


def test_token_rows_with_a_stride_and_errors():
    from longlive_b200 import ops
    C, f, h, w = 4, 2, 3, 5
    lat = torch.randn(C, f, 2 * h, 2 * w, device="cuda").bfloat16()
    wide = torch.full((f * h * w, 4 * C + 8), 3.0, device="cuda", dtype=torch.bfloat16)
    ops.patchify(lat, out=wide[:, :4 * C])
    assert torch.equal(wide[:, :4 * C], _ref_patchify(lat)) and bool((wide[:, 4 * C:] == 3).all())
    with pytest.raises(RuntimeError):
        ops.patchify(lat[:, :, :, ::2])
    with pytest.raises(RuntimeError):
        ops.patchify(lat.float())
    with pytest.raises(RuntimeError):
        ops.unpatchify(wide, torch.empty_like(lat))


def test_handoff_to_pinned_host_in_order_with_backpressure():
    from longlive_b200 import ops
    from longlive_b200.handoff import LatentHandoff
    C, f, h, w = 48, 3, 22, 40
    ho = LatentHandoff(C, f, 2 * h, 2 * w, depth=2)
    g = torch.Generator(device="cuda").manual_seed(1)
    lats = [torch.randn(C, f, 2 * h, 2 * w, device="cuda", generator=g).bfloat16() for _ in range(5)]
    toks = [ops.patchify(x) for x in lats]
    assert ho.pop() is None
    assert ho.push(toks[0]) == 0 and ho.push(toks[1]) == 1
    with pytest.raises(RuntimeError):
        ho.push(toks[2])                                   # ring of two: chunk 0 has not been released
    seq, host = ho.pop()
    assert seq == 0 and host.is_pinned() and torch.equal(host, lats[0].cpu())
    ho.release(0)
    assert ho.push(toks[2]) == 2
    for want in (1, 2):
        seq, host = ho.pop()
        assert seq == want and torch.equal(host, lats[want].cpu())
        ho.release(seq)
    assert ho.pop(wait=False) is None and ho.bytes_per_chunk == C * f * 4 * h * w * 2


def test_handoff_does_not_block_the_compute_stream():
    """The copies run on their own stream: work queued on the compute stream after push() does not wait for them."""
    from longlive_b200 import ops
    from longlive_b200.handoff import LatentHandoff
    C, f, h, w = 48, 3, 22, 40
    ho = LatentHandoff(C, f, 2 * h, 2 * w, depth=3)
    tok = ops.patchify(torch.randn(C, f, 2 * h, 2 * w, device="cuda").bfloat16())
    for i in range(3):
        ho.push(tok)
    torch.cuda.current_stream().synchronize()              # returns once the unpatchify kernels are done ...
    for i in range(3):
        seq, host = ho.pop()                               # ... the copies are waited for here
        assert seq == i
        ho.release(seq)
