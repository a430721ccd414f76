"""CUDA-graph capture and replay of the operator, and calls on a device that is not the current one
(reference: tests/attention/triangle/test_triangle_attention.py:295-304 secondary device, :454-508 ragged forward +
backward capture cold and warm, :536-555 dense capture)."""

from __future__ import annotations

import gc

import pytest
import torch

from oops_b200 import triangle_attention
from test_triangle_gpu import (
    assert_within, build_nested, dense_case, nested_case, nested_oracle, oracle_dense, to_device,
)

pytestmark = pytest.mark.gpu


def _captured(call, stream, warm_calls):
    """Warm up, capture `call` into a graph on `stream` and return (graph, captured results)."""
    with torch.cuda.stream(stream):
        for warm in warm_calls:
            warm()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            captured = call()
    return graph, captured


def test_graph_forward_backward_on_the_tensor_kernels(cuda):
    """Forward and all four gradients of a 16-bit head-size-32 call (tcgen05 kernels, scratch allocated inside the
    capture) replayed on changed inputs."""
    case = dense_case(torch.bfloat16, prefix=(1,), rows=6, cols=200, heads=4, dim=32, bias_kind="shared", scale_inputs=0.5)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        args, leaves = to_device(case, cuda)
        upstream = case["upstream"].to(cuda)
    wanted = [leaves[n] for n in ("q", "k", "v", "bias")]

    def call():
        out = triangle_attention(args["q"], args["k"], args["v"], args["mask"], args["bias"])
        return (out, *torch.autograd.grad(out, wanted, upstream))

    graph, captured = _captured(call, stream, [call] * 3)
    with torch.cuda.stream(stream), torch.no_grad():
        other = dense_case(torch.bfloat16, prefix=(1,), rows=3, cols=72, heads=4, dim=32, bias_kind="none", scale_inputs=0.5)
        other_args, _ = to_device(other, cuda, active=())
        triangle_attention(other_args["q"], other_args["k"], other_args["v"], other_args["mask"], None)
        del other_args
        gc.collect()
        leaves["q"].mul_(0.5)
        graph.replay()
    stream.synchronize()
    case["q"] = (case["q"].float() * 0.5).to(torch.bfloat16)
    want = oracle_dense(case)
    assert_within(captured[0], want[0], 2e-2, "out")
    for name, got, ref in zip(("dq", "dk", "dv", "dbias"), captured[1:], want[1:]):
        assert_within(got, ref, 2e-2 * max(1.0, float(ref.abs().max())), name)


@pytest.mark.parametrize("warm,dim,only_bias", [(False, 24, False), (True, 24, True), (False, 129, True), (True, 129, False)])
def test_graph_ragged_forward_backward(cuda, warm, dim, only_bias):
    """A packed ragged batch, forward + backward, captured cold (first call with these lengths is the capture) or
    warm, with other shapes run between capture and replay."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    prefix = (2,) if warm else ()
    with torch.cuda.stream(stream):
        other_case = nested_case(torch.float32, cuda, lengths=(19, 17), dim=dim, bias_kind="shared", prefix=prefix, seed=3)
        other = build_nested(other_case, cuda)
        case = nested_case(torch.float32, cuda, lengths=(17, 19), dim=dim, bias_kind="shared", prefix=prefix, seed=4)
        q, k, v, mask, bias, leaves = build_nested(case, cuda)
        upstream = torch.randn(leaves["q"].shape, generator=torch.Generator().manual_seed(9)).to(cuda)
    names = ("bias",) if only_bias else ("q", "k", "v", "bias")

    def run(inputs, inputs_leaves):
        values = triangle_attention(*inputs[:5]).concat
        return (values, *torch.autograd.grad(values, [inputs_leaves[n] for n in names], upstream))

    warm_calls = [lambda: run(other, other[5])] * 3 + ([lambda: run((q, k, v, mask, bias), leaves)] if warm else [])
    graph, captured = _captured(lambda: run((q, k, v, mask, bias), leaves), stream, warm_calls)
    with torch.cuda.stream(stream), torch.no_grad():
        for lengths in ((11, 7), (23, 13)):
            extra = build_nested(nested_case(torch.float32, cuda, lengths=lengths, dim=24, bias_kind="none"), cuda, False)
            triangle_attention(*extra[:5])
            del extra
        gc.collect()
        leaves["q"].add_(0.1)
        graph.replay()
    stream.synchronize()
    case["elements"]["q"] = [e + 0.1 for e in case["elements"]["q"]]
    compute = torch.float64 if dim > 128 else torch.float32
    want_out, want = nested_oracle(case, upstream.cpu(), compute)
    assert_within(captured[0], want_out, 1e-4, "out")
    for name, got in zip(names, captured[1:]):
        assert_within(got, want[name], 1e-4 * max(1.0, float(want[name].abs().max())), f"d{name}")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_second_device_while_another_is_current():
    """Operands on cuda:1 while cuda:0 is the current device: kernels, scratch and streams follow the operands."""
    device = torch.device("cuda", 1)
    assert torch.cuda.current_device() == 0
    for dtype, dim in ((torch.float32, 24), (torch.bfloat16, 32)):
        case = dense_case(dtype, dim=dim, cols=72, bias_kind="shared", scale_inputs=0.5)
        args, leaves = to_device(case, device)
        out = triangle_attention(args["q"], args["k"], args["v"], args["mask"], args["bias"])
        assert out.device == device
        grads = torch.autograd.grad(out, [leaves[n] for n in ("q", "k", "v", "bias")], case["upstream"].to(device))
        want = oracle_dense(case)
        atol = 1e-4 if dtype is torch.float32 else 2e-2
        assert_within(out, want[0], atol, "out")
        for name, got, ref in zip(("dq", "dk", "dv", "dbias"), grads, want[1:]):
            assert got.device == device
            assert_within(got, ref, atol * max(1.0, float(ref.abs().max())), name)
    assert torch.cuda.current_device() == 0
