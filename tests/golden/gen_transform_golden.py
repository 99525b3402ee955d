"""Generates tests/golden/transform_golden.npz from the reference's OWN runtime tensor transforms.

Run in a container that has the reference checkout:

    python tests/golden/gen_transform_golden.py /path/to/tt-buda

The functions are taken straight out of the reference's source files -- `_embedding_index`, `is_buda_shape` and
`pad_pytorch_tensor_to_buda` from pybuda/pybuda/tensor.py, `eval` (its "conv2d_prestride_act" branch) from
pybuda/pybuda/op/eval/pybuda/tm.py -- by parsing the file and executing only those definitions: the modules around
them cannot be imported (tensorflow, jax, the unbuilt pybuda._C).  The few names the definitions use are supplied here.
Inputs and outputs are stored together, so the fixture does not depend on any random generator afterwards.
"""
import ast
import os
import sys
import types
import typing

import numpy as np
import torch


def _definitions(path, names, namespace):
    """Executes the named top-level function definitions of a source file inside `namespace`."""
    with open(path) as f:
        tree = ast.parse(f.read(), filename=path)
    picked = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    assert {n.name for n in picked} == set(names), (path, names)
    exec(compile(ast.Module(body=picked, type_ignores=[]), path, "exec"), namespace)
    return [namespace[n] for n in names]


def load_reference(ref_root):
    df = types.SimpleNamespace(RawUInt8="RawUInt8", RawUInt16="RawUInt16", RawUInt32="RawUInt32")
    ns = {"torch": torch, "TILE_DIM": 32, "align_up": lambda v, a: (v + a - 1) // a * a, "DataFormat": df, "DramIODesc": object,
          "Tuple": typing.Tuple, "List": typing.List, "Optional": typing.Optional, "Union": typing.Union,
          "to_torch_operands": lambda *a: a}
    emb, _, pad = _definitions(os.path.join(ref_root, "pybuda/pybuda/tensor.py"),
                               ["_embedding_index", "is_buda_shape", "pad_pytorch_tensor_to_buda"], ns)
    (tm_eval,) = _definitions(os.path.join(ref_root, "pybuda/pybuda/op/eval/pybuda/tm.py"), ["eval"], dict(ns))
    return emb, pad, tm_eval, df


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: gen_transform_golden.py <path of a tt-buda checkout>")
    emb, pad, tm_eval, df = load_reference(sys.argv[1])
    g = torch.Generator().manual_seed(11)
    out = {}

    # ---- embedding index: (indices per entry, entries, queue tile rows, queue tile columns)
    for k, (n, w, q_rt, q_ct) in enumerate([(100, 1, 1, 1), (1024, 1, 1, 1), (2040, 2, 2, 1), (3050, 3, 3, 1), (37, 1, 1, 1)]):
        idx = torch.randint(0, 50000, (w, n) if w > 1 else (n,), generator=g, dtype=torch.int32)
        q = types.SimpleNamespace(data_format=df.RawUInt32, bufq_grid_dim_r=1, mblock_m=q_rt, ublock_rt=1, t=1,
                                  bufq_grid_dim_c=1, mblock_n=q_ct, ublock_ct=1)
        res = emb(idx.clone(), (n,), q)
        out[f"emb{k}_in"] = idx.numpy()
        out[f"emb{k}_meta"] = np.array([n, w, q_rt, q_ct])
        out[f"emb{k}_out"] = res.contiguous().numpy()

    # ---- padding to tiles: (shape, tile-broadcast dims)
    for k, (shape, bcast) in enumerate([((1, 3, 50, 70), []), ((2, 1, 1, 40), [2]), ((1, 2, 33, 1), [3]), ((4, 17), []), ((1, 1, 64, 64), [])]):
        x = torch.randn(shape, generator=g)
        res = pad(x, bcast, squeeze=True, microbatch=shape[0] if len(shape) == 4 else 1)
        out[f"pad{k}_in"] = x.numpy()
        out[f"pad{k}_bcast"] = np.array(bcast, dtype=np.int64)
        out[f"pad{k}_out"] = res.contiguous().numpy()

    # ---- convolution activation prestride (golden of the push-time transform): (shape, stride)
    for k, (shape, s) in enumerate([((1, 3, 8, 8), 2), ((2, 4, 9, 7), 2), ((1, 2, 10, 10), 3), ((1, 16, 32, 30), 4)]):
        act = torch.randn(shape, generator=g)
        res = tm_eval("conv2d_prestride_act", [s, s, 3, 3, shape[2], shape[3]], [act])
        out[f"pre{k}_in"] = act.numpy()
        out[f"pre{k}_stride"] = np.array([s])
        out[f"pre{k}_out"] = res.contiguous().numpy()

    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "transform_golden.npz"), **out)
    print(sorted(out), "written")


if __name__ == "__main__":
    main()
