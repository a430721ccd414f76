"""Generate the golden vectors under tests/golden/ from the reference's own code.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

The reference test module cannot be imported as a whole here (it imports the
third-party ``danling`` package, which is absent), so the two pure-PyTorch
functions that pin the operator's results, ``_reference`` and
``_flatten_nested_attention`` in
``tests/attention/triangle/test_triangle_attention.py`` (:42-58, :160-169), are
taken out of the file's syntax tree and executed unchanged.  Their outputs and
autograd gradients on seeded inputs are written as ``*.pt`` files, inputs
included, so that the files stand alone where the reference is not present.
"""

from __future__ import annotations

import ast
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
WANTED = ("_reference", "_flatten_nested_attention")


def load_reference_functions(reference_root: Path):
    source_path = reference_root / "tests" / "attention" / "triangle" / "test_triangle_attention.py"
    tree = ast.parse(source_path.read_text())
    picked = [node for node in tree.body if isinstance(node, ast.FunctionDef) and node.name in WANTED]
    assert {node.name for node in picked} == set(WANTED), "reference test file changed"
    module = ast.Module(body=picked, type_ignores=[])
    namespace = {"torch": torch}
    exec(compile(module, str(source_path), "exec"), namespace)
    return namespace["_reference"], namespace["_flatten_nested_attention"]


def grads_of(reference, q, k, v, mask, bias, upstream, compute_dtype):
    leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]
    bias_leaf = None if bias is None else bias.detach().clone().requires_grad_(True)
    out = reference(leaves[0], leaves[1], leaves[2], mask, bias_leaf, compute_dtype=compute_dtype)
    wanted = leaves + ([] if bias_leaf is None else [bias_leaf])
    grads = torch.autograd.grad(out, wanted, upstream.to(out.dtype))
    return out.detach(), grads


def dense_case(reference, name, *, seed, prefix, rows, cols, heads, dim, dtype, bias_kind, mask_kind, compute_dtype):
    gen = torch.Generator().manual_seed(seed)
    shape = (*prefix, rows, cols, heads, dim)
    q, k, v = (torch.randn(shape, generator=gen).to(dtype) for _ in range(3))
    bias = None
    if bias_kind != "none":
        groups = 1 if bias_kind == "shared" else rows
        bias = torch.randn((*prefix, groups, heads, cols, cols), generator=gen).to(dtype)
    mask = None
    if mask_kind != "none":
        mask = torch.rand((*prefix, rows, cols), generator=gen) > 0.2
        mask[..., 0] = True
        if mask_kind == "row0_empty":
            mask[..., 0, :] = False
    upstream = torch.randn(shape, generator=gen)
    out, grads = grads_of(reference, q, k, v, mask, bias, upstream, compute_dtype)
    record = {
        "name": name, "compute_dtype": str(compute_dtype), "q": q, "k": k, "v": v, "mask": mask, "bias": bias,
        "upstream": upstream, "out": out, "dq": grads[0], "dk": grads[1], "dv": grads[2],
        "dbias": grads[3] if bias is not None else None,
    }
    torch.save(record, HERE / f"{name}.pt")
    print(name, tuple(out.shape), float(out.abs().max()))


def config1_case(reference):
    """BASELINE config 1 (fp32, B=1, N=64, H=4, D=32).  Inputs are regenerated
    from the seed by the consumer; a checksum guards the generator, and the
    outputs are stored on a stride-4 lattice of the pair axes to stay small."""
    gen = torch.Generator().manual_seed(0)
    n, h, d = 64, 4, 32
    q, k, v = (torch.randn(1, n, n, h, d, generator=gen) for _ in range(3))
    bias = torch.randn(1, 1, h, n, n, generator=gen)
    upstream = torch.randn(1, n, n, h, d, generator=gen)
    mask = torch.ones(1, n, n, dtype=torch.bool)
    out, grads = grads_of(reference, q, k, v, mask, bias, upstream, torch.float32)
    lattice = (slice(None), slice(None, None, 4), slice(None, None, 4))
    record = {
        "name": "config1", "seed": 0, "n": n, "heads": h, "dim": d,
        "input_checksum": torch.stack([t.double().sum() for t in (q, k, v, bias, upstream)]),
        "out": out[lattice].clone(), "dq": grads[0][lattice].clone(), "dk": grads[1][lattice].clone(),
        "dv": grads[2][lattice].clone(), "dbias": grads[3][..., ::2, ::2].clone(),
    }
    torch.save(record, HERE / "config1.pt")
    print("config1", tuple(record["out"].shape))


def nested_case(reference, flatten):
    gen = torch.Generator().manual_seed(3)
    heads, dim, lengths = 2, 16, (3, 5)
    elements, outs = [], []
    for n in lengths:
        q, k, v = (torch.randn(n, n, heads, dim, generator=gen) for _ in range(3))
        bias = torch.randn(1, heads, n, n, generator=gen)
        mask = torch.rand(n, n, generator=gen) > 0.2
        mask[:, 0] = True
        elements.append({"q": q, "k": k, "v": v, "bias": bias, "mask": mask})
        outs.append(reference(q, k, v, mask, bias))
    record = {
        "name": "nested", "lengths": lengths, "elements": elements,
        "packed": flatten(outs), "packed_transposed": flatten(outs, transposed_pair_axes=True),
    }
    torch.save(record, HERE / "nested.pt")
    print("nested", tuple(record["packed"].shape))


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference>")
    reference_root = Path(sys.argv[1])
    reference, flatten = load_reference_functions(reference_root)
    dense_case(reference, "dense_f32_shared_masked", seed=1, prefix=(2,), rows=4, cols=33, heads=2, dim=24,
               dtype=torch.float32, bias_kind="shared", mask_kind="random", compute_dtype=torch.float32)
    dense_case(reference, "dense_f64_full_row0_empty", seed=117, prefix=(1,), rows=17, cols=17, heads=2, dim=9,
               dtype=torch.float32, bias_kind="full", mask_kind="row0_empty", compute_dtype=torch.float64)
    dense_case(reference, "dense_f32_plain", seed=5, prefix=(1,), rows=3, cols=40, heads=1, dim=32,
               dtype=torch.float32, bias_kind="none", mask_kind="none", compute_dtype=torch.float32)
    dense_case(reference, "dense_bf16_shared", seed=7, prefix=(1,), rows=3, cols=40, heads=4, dim=32,
               dtype=torch.bfloat16, bias_kind="shared", mask_kind="random", compute_dtype=torch.float32)
    config1_case(reference)
    nested_case(reference, flatten)


if __name__ == "__main__":
    main()
