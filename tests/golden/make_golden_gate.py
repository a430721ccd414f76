"""Generates tests/golden/gate.pt from the reference's own PyTorch statement of gate_attention_output.

    python tests/golden/make_golden_gate.py /path/to/reference

The reference test module cannot be imported here (it needs DanLing), so `_reference` is lifted out of
tests/attention/gate/test_gate_attention_output.py by its syntax tree and run unchanged on seeded inputs; inputs,
output and autograd gradients are stored.
"""

from __future__ import annotations

import ast
import sys
from pathlib import Path

import torch
from torch.nn import functional as F


def lift_reference(reference_root: Path):
    source = (reference_root / "tests" / "attention" / "gate" / "test_gate_attention_output.py").read_text()
    tree = ast.parse(source)
    wanted = [node for node in tree.body if isinstance(node, ast.FunctionDef) and node.name == "_reference"]
    assert len(wanted) == 1
    namespace = {"torch": torch, "F": F}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), "reference_gate", "exec"), namespace)  # noqa: S102
    return namespace["_reference"]


def main():
    reference = lift_reference(Path(sys.argv[1]))
    cases = {}
    for name, dtype, shape in (("f32_rank4", torch.float32, (2, 4, 37, 16)), ("f64_rank3", torch.float64, (3, 9, 8)),
                               ("f32_rank5", torch.float32, (2, 3, 2, 11, 32))):
        gen = torch.Generator().manual_seed(71)
        *prefix, heads, length, head_size = shape
        channels, single_channels, out_channels = heads * head_size, 12, 7
        attention = torch.randn(shape, generator=gen, dtype=dtype, requires_grad=True)
        single = torch.randn(*prefix, length, single_channels, generator=gen, dtype=dtype, requires_grad=True)
        gate_weight = (torch.randn(channels, single_channels, generator=gen, dtype=dtype) / single_channels**0.5).requires_grad_(True)
        output_weight = (torch.randn(out_channels, channels, generator=gen, dtype=dtype) / 8).requires_grad_(True)
        out = reference(attention, single, gate_weight, output_weight)
        upstream = torch.randn(out.shape, generator=gen, dtype=dtype)
        grads = torch.autograd.grad(out, (attention, single, gate_weight, output_weight), upstream)
        cases[name] = dict(
            attention=attention.detach(), single=single.detach(), gate_weight=gate_weight.detach(),
            output_weight=output_weight.detach(), upstream=upstream, out=out.detach(),
            grads=[g.detach() for g in grads],
        )
    torch.save(cases, Path(__file__).resolve().parent / "gate.pt")
    print("wrote gate.pt:", {k: tuple(v["out"].shape) for k, v in cases.items()})


if __name__ == "__main__":
    main()
