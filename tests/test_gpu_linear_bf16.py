"""The bf16 Linear kernel of the unquantized edge layers (llnv_linear_bf16) against an fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(x, w, b, act):
    y = x.float() @ w.float().t()
    if b is not None:
        y = y + b.float()
    if act is not None:
        y = y.bfloat16().float()                      # the reference's activation is a separate op on the bf16 result
        y = torch.nn.functional.gelu(y, approximate="tanh") if act == "gelu_tanh" else torch.nn.functional.silu(y)
    return y


def _check(x, w, b, act, out):
    """fp32 accumulation in another order, then one bf16 rounding (two with an activation)."""
    ref = _ref(x, w, b, act)
    k = x.shape[1]
    mag = (x.float().abs() @ w.float().abs().t()) + (0 if b is None else b.float().abs())
    tol = ref.abs() * 2.0 ** -7 + mag * (k * 2.0 ** -24) + 1e-30
    if act is not None:
        tol = tol + (ref.abs() + mag.clamp(max=1.0)) * 2.0 ** -6
    err = (out.float() - ref).abs()
    assert bool((err <= tol).all()), f"max err {float(err.max())} at tol {float(tol.flatten()[err.argmax()])}"


# the edge layers of the DiT: patch embedding, head, text embedding (both Linears), time embedding / projection
SHAPES = [(2640, 3072, 192, None), (2640, 192, 3072, None), (512, 3072, 4096, "gelu_tanh"), (512, 3072, 3072, None),
          (3, 3072, 256, "silu"), (3, 18432, 3072, None), (330, 192, 3072, None)]


@pytest.mark.parametrize("m,n,k,act", SHAPES)
def test_edge_layer_shapes(m, n, k, act):
    from longlive_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    x = torch.randn(m, k, device="cuda", generator=g).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) * k ** -0.5).bfloat16()
    b = torch.randn(n, device="cuda", generator=g).bfloat16()
    out = ops.linear_bf16(x, w, b, act)
    _check(x, w, b, act, out)
    assert torch.equal(out, ops.linear_bf16(x, w, b, act))                          # deterministic


@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (127, 40, 72), (129, 136, 200), (257, 64, 64), (300, 200, 1000)])
def test_ragged_sizes_strides_and_no_bias(m, n, k):
    """M, N, K off the tile sizes (TMA zero fill, masked stores), strided input rows, output into a wider buffer."""
    from longlive_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(7)
    xb = torch.randn(m, k + 16, device="cuda", generator=g).bfloat16()
    x = xb[:, 8:8 + k]                                                             # row stride k + 16, 16-byte aligned start
    w = (torch.randn(n, k, device="cuda", generator=g) * k ** -0.5).bfloat16()
    buf = torch.full((m, n + 24), 7.0, device="cuda", dtype=torch.bfloat16)
    out = ops.linear_bf16(x, w, None, None, out=buf[:, 8:8 + n])
    _check(x, w, None, None, out)
    assert bool((buf[:, :8] == 7).all()) and bool((buf[:, 8 + n:] == 7).all())      # nothing written outside


def test_rows_do_not_depend_on_the_row_count():
    """A row's result does not depend on how many rows the call has (token shards of a sequence-parallel run)."""
    from longlive_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(2640, 3072, device="cuda", generator=g).bfloat16()
    w = (torch.randn(192, 3072, device="cuda", generator=g) * 0.02).bfloat16()
    full = ops.linear_bf16(x, w)
    for lo, hi in ((0, 330), (330, 660), (1320, 2640)):
        assert torch.equal(full[lo:hi], ops.linear_bf16(x[lo:hi], w))


def test_argument_errors():
    from longlive_b200 import ops
    x = torch.zeros(4, 16, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(8, 16, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.linear_bf16(x, w, act="relu")
    with pytest.raises(RuntimeError):
        ops.linear_bf16(x.float(), w)
    with pytest.raises(RuntimeError):
        ops.linear_bf16(x, w[:, :8].contiguous())
    with pytest.raises(RuntimeError):
        ops.linear_bf16(x[:, :12], w[:, :12])                                      # K not a multiple of 8
    assert ops.linear_bf16(x[:0], w).shape == (0, 8)
