"""Argument checking and error conventions that need no GPU
(reference: tests/attention/triangle/test_triangle_attention.py:509-581 scenarios cpu/shape/dtype/forward_ad/nested_shape)."""

from __future__ import annotations

import pytest
import torch
from torch.autograd import forward_ad

from oops_b200 import NestedTensor, OOpsUnsupportedError, triangle_attention
from oops_b200.attention.triangle.function import NestedGeometry
from oracle import triangle_oracle as oracle


def _dense(dtype=torch.float32):
    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 4, 9, 2, 8, dtype=dtype) for _ in range(3))
    mask = torch.rand(2, 4, 9) > 0.2
    bias = torch.randn(2, 1, 2, 9, 9, dtype=dtype)
    return q, k, v, mask, bias


def test_cpu_tensors_are_unsupported():
    with pytest.raises(OOpsUnsupportedError, match="triangle_attention requires CUDA"):
        triangle_attention(*_dense())
    assert issubclass(OOpsUnsupportedError, NotImplementedError)


def test_shape_mismatch_is_value_error():
    q, k, v, mask, bias = _dense()
    with pytest.raises(ValueError):
        triangle_attention(q, k, v[..., :-1], mask, bias)
    with pytest.raises(ValueError):
        triangle_attention(q, k, v, mask[:, :3], bias)
    with pytest.raises(ValueError):
        triangle_attention(q, k, v, mask, bias[:, :, :1])
    with pytest.raises(ValueError):
        triangle_attention(q[0, 0], k[0, 0], v[0, 0])


def test_double_is_unsupported():
    q, k, v, mask, bias = _dense(torch.float64)
    with pytest.raises(OOpsUnsupportedError):
        triangle_attention(q, k, v, mask, bias)


def test_non_bool_mask_is_unsupported():
    q, k, v, mask, bias = _dense()
    with pytest.raises(OOpsUnsupportedError, match="bool keep-mask"):
        triangle_attention(q, k, v, mask.to(torch.int32), bias)


def test_forward_mode_is_rejected():
    q, k, v, mask, bias = _dense()
    with forward_ad.dual_level():
        dual = forward_ad.make_dual(q, torch.ones_like(q))
        with pytest.raises(OOpsUnsupportedError, match="forward-mode"):
            triangle_attention(dual, k, v, mask, bias)


def test_mixed_dense_nested_is_value_error():
    q, k, v, mask, bias = _dense()
    nested = NestedTensor([torch.randn(3, 3, 2, 8)], ragged_dims=(0, 1))
    with pytest.raises(ValueError):
        triangle_attention(nested, k, v)
    with pytest.raises(ValueError):
        triangle_attention(q, nested, v)
    with pytest.raises(ValueError):
        triangle_attention(q, k, v, nested)


def test_non_square_nested_is_value_error():
    q = NestedTensor([torch.randn(2, 3, 2, 24)], ragged_dims=(0, 1))
    with pytest.raises(ValueError):
        triangle_attention(q, q, q)


def test_nested_geometry_views_match_unbind():
    """The per-sample strided views of the packed layout address the same elements as unbind()."""
    torch.manual_seed(1)
    lengths, prefix, heads, dim = (3, 5, 4), (2,), 2, 4
    elements = [torch.randn(*prefix, n, n, heads, dim) for n in lengths]
    nested = NestedTensor(elements, ragged_dims=(1, 2))
    for transposed in (False, True):
        view = nested.transpose(-4, -3) if transposed else nested
        packed = view.concat.reshape(view.concat.shape[0], 2, heads, dim).contiguous()
        geometry = NestedGeometry(lengths=lengths, prefixes=2, transposed=transposed)
        for got, want in zip(geometry.pair_views(packed), torch.unbind(view)):
            torch.testing.assert_close(got, want, atol=0, rtol=0)
        if transposed:
            for got, original in zip(geometry.pair_views(packed), elements):
                torch.testing.assert_close(got, original.transpose(1, 2), atol=0, rtol=0)


def test_nested_packing_matches_oracle_flatten():
    torch.manual_seed(2)
    elements = [torch.randn(n, n, 2, 4) for n in (3, 5)]
    nested = NestedTensor(elements, ragged_dims=(0, 1))
    torch.testing.assert_close(nested.concat, oracle.flatten_nested(elements), atol=0, rtol=0)
    swapped = nested.transpose(-4, -3)
    assert swapped.ragged_dims == (1, 0) and swapped.packed_dim_order == (1, 0, 2, 3)
    torch.testing.assert_close(
        swapped.concat, oracle.flatten_nested(torch.unbind(swapped), transposed_pair_axes=True), atol=0, rtol=0
    )


def test_fake_tensors_take_the_dispatcher_route():
    """Shapes and dtypes come from the registered fake implementations; no kernel runs
    (reference: tests/attention/triangle/test_triangle_attention.py:556-559)."""
    from torch._subclasses.fake_tensor import FakeTensorMode, is_fake

    with FakeTensorMode(allow_non_fake_inputs=True):
        q = torch.empty(2, 4, 37, 2, 24, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        swapped = torch.empty(2, 37, 4, 2, 24, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
        bias = torch.empty(2, 1, 2, 37, 37, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        mask = torch.empty(2, 4, 37, device="cuda", dtype=torch.bool)
        out = triangle_attention(q, swapped, swapped, mask, bias)
        plain = triangle_attention(q.detach(), swapped, swapped)
    assert is_fake(out) and out.shape == q.shape and out.dtype == torch.bfloat16 and out.device.type == "cuda"
    assert out.requires_grad  # the reverse pass of fake CUDA tensors needs a device: covered by the GPU suite
    assert is_fake(plain) and not plain.requires_grad


def test_fake_nested_keeps_the_packing():
    from torch._subclasses.fake_tensor import FakeTensorMode, is_fake

    with FakeTensorMode(allow_non_fake_inputs=True):
        q = NestedTensor([torch.empty(n, n, 2, 16, device="cuda") for n in (3, 5)], ragged_dims=(0, 1))
        bias = NestedTensor([torch.empty(1, 2, n, n, device="cuda") for n in (3, 5)], ragged_dims=(2, 3))
        out = triangle_attention(q, q, q, None, bias)
    assert is_fake(out.concat) and out.concat.shape == (34, 2, 16) and out.ragged_dims == q.ragged_dims


def test_geometry_survives_the_integer_encoding():
    from oops_b200.attention.triangle.function import DenseGeometry, decode_geometry, encode_geometry

    nested = NestedGeometry(lengths=(3, 5), prefixes=2, transposed=True, bias_groups=(1, 5), bias_row_strides=(8, 8))
    assert decode_geometry(encode_geometry(nested)) == nested
    plain = NestedGeometry(lengths=(7,), prefixes=1, transposed=False)
    assert decode_geometry(encode_geometry(plain)) == plain
    assert decode_geometry(encode_geometry(DenseGeometry())) == DenseGeometry()
