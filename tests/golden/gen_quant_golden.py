"""Generates tests/golden/quant_golden.npz from the reference's OWN golden quantise ops.

Run in a container that has the reference checkout:

    python tests/golden/gen_quant_golden.py /path/to/tt-buda

It loads pybuda/pybuda/op/eval/pybuda/quantize.py (eval, lines 55-122) and
pybuda/pybuda/op/eval/buda/quantize.py (eval, lines 23-53) straight from their files; the
package around them cannot be imported (it pulls in tensorflow, jax and the unbuilt pybuda._C),
so the handful of names those two files import are provided as empty stub modules.  Inputs and
outputs are stored together, so the fixture does not depend on any random generator afterwards.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch


def _stub(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    m.__path__ = []
    sys.modules[name] = m
    return m


def load_reference(ref_root):
    class _Anything:
        def __getattr__(self, k):
            return _Anything()

        def __call__(self, *a, **k):
            return _Anything()

    _stub("pybuda")
    _stub("pybuda.pybudaglobal", TILE_DIM=32)
    _stub("pybuda.utils", align_up_tile=lambda v: (v + 31) // 32 * 32, align_up=lambda v, a: (v + a - 1) // a * a)
    _stub("pybuda.tensor", pytorch_dtype_to_buda_dataformat=lambda *a, **k: None)
    _stub("pybuda._C", DataFormat=_Anything(), MathFidelity=_Anything())
    _stub("pybuda._C.balancer")
    _stub("pybuda._C.backend_api", get_op_model_execution_cycles=lambda *a, **k: 0)
    _stub("pybuda._C.graph", UBlockOrder=_Anything())
    _stub("loguru", logger=_Anything())
    _stub("pybuda.op")
    _stub("pybuda.op.eval")
    _stub("pybuda.op.eval.common", to_torch_operands=lambda *a: a, op_model_to_desc=None,
          get_compiler_cached_cycles=None)
    _stub("pybuda.op.eval.pybuda")
    _stub("pybuda.op.eval.pybuda.reciprocal", Reciprocal=object)
    _stub("pybuda.op.eval.buda")

    def load(modname, rel):
        spec = importlib.util.spec_from_file_location(modname, os.path.join(ref_root, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[modname] = mod
        spec.loader.exec_module(mod)
        return mod

    py = load("pybuda.op.eval.pybuda.quantize", "pybuda/pybuda/op/eval/pybuda/quantize.py")
    bu = load("pybuda.op.eval.buda.quantize", "pybuda/pybuda/op/eval/buda/quantize.py")
    return py, bu


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: gen_quant_golden.py <path of a tt-buda checkout>")
    ref_root = sys.argv[1]
    py, bu = load_reference(ref_root)
    g = torch.Generator(device="cpu")
    out = {}

    # ---- case A: per-tensor Quantize / Dequantize, the shape class of the int8 config: U(-6,6),
    # scale 0.05, zero point 3; plus values that saturate and exact .5 ties.
    g.manual_seed(3)
    x = torch.rand(8, 16, 64, generator=g) * 12 - 6
    x.view(-1)[:8] = torch.tensor([0.025, 0.075, -0.025, -0.075, 6.5, -6.6, 1e9, -1e9])
    scale = torch.tensor([0.05])
    q = py.eval("quantize", (3, -1, "torch.int8"), [x, scale])
    dq = py.eval("dequantize", (3, -1), [q, scale])
    out.update(a_x=x, a_scale=scale, a_zp=np.float32(3), a_q=q, a_dq=dq)
    # float zero point, as the front-end emits it
    q2 = py.eval("quantize", (3.0, -1, "torch.int8"), [x, scale])
    assert torch.equal(q, q2)

    # ---- case B: per-axis Quantize / Dequantize on the last and on a middle axis
    g.manual_seed(13)
    xb = torch.randn(4, 24, 40, generator=g) * 3
    sb_last = torch.rand(40, generator=g) * 0.09 + 0.01
    sb_mid = torch.rand(24, generator=g) * 0.09 + 0.01
    qb_last = py.eval("quantize", (-5, -1, "torch.int8"), [xb, sb_last])
    qb_mid = py.eval("quantize", (7, 1, "torch.int8"), [xb, sb_mid])
    dqb_last = py.eval("dequantize", (-5, -1), [qb_last, sb_last])
    dqb_mid = py.eval("dequantize", (7, 1), [qb_mid, sb_mid])
    out.update(b_x=xb, b_scale_last=sb_last, b_scale_mid=sb_mid, b_q_last=qb_last, b_q_mid=qb_mid,
               b_dq_last=dqb_last, b_dq_mid=dqb_mid)

    # ---- case C: BudaQuantize / buda "quantization" (multiply by a reciprocal scale, pre-broadcast)
    rb = (1.0 / sb_last).reshape(1, 1, 40).broadcast_to(xb.shape).contiguous()
    qc = py.eval("buda_quantize", (2, -1, "torch.int8"), [xb, rb])
    qc2 = bu.eval("quantization", (2, -1, "torch.int8"), [xb, rb])
    assert torch.equal(qc, qc2)
    dqc = bu.eval("dequantization", (2, -1), [qc, sb_last.reshape(1, 1, 40).broadcast_to(xb.shape).contiguous()])
    out.update(c_recip=rb, c_q=qc, c_dq=dqc)

    # ---- case D: Requantize from int32 accumulators ~U(-2^20, 2^20), per-channel scales
    # ~U(1e-4, 1e-2) on the last axis, zero point 0 (and a non-zero output zero point)
    g.manual_seed(4)
    acc = torch.randint(-2 ** 20, 2 ** 20, (6, 32, 128), generator=g, dtype=torch.int32)
    acc.view(-1)[:6] = torch.tensor([2 ** 31 - 1, -2 ** 31, 16777217, -16777219, 0, 1], dtype=torch.int32)
    g.manual_seed(5)
    scales = torch.rand(128, generator=g) * (1e-2 - 1e-4) + 1e-4
    ones = torch.ones(128)
    rq = py.eval("requantize", (0, 0, -1, "None", "torch.int8"), [acc, scales, ones])
    rq_zp = py.eval("requantize", (11, 0, -1, "None", "torch.int8"), [acc, scales, ones])
    out_scale = torch.rand(128, generator=g) * 0.5 + 0.5
    rq_div = py.eval("requantize", (-3, 0, -1, "None", "torch.int8"), [acc, scales, out_scale])
    sc_b = scales.reshape(1, 1, 128).broadcast_to(acc.shape).contiguous()
    brq = py.eval("buda_requantize", (0, -1, "None", "torch.int8"), [acc, sc_b])
    brq2 = bu.eval("requantization", (0,), [acc, sc_b])
    assert torch.equal(brq, brq2)
    assert torch.equal(brq, rq)  # inp_scale / 1 == inp_scale
    # requantize along a middle axis
    sc_mid = torch.rand(32, generator=g) * (1e-2 - 1e-4) + 1e-4
    rq_mid = py.eval("requantize", (5, 0, 1, "None", "torch.int8"), [acc, sc_mid, torch.ones(32)])
    out.update(d_acc=acc, d_scales=scales, d_out_scale=out_scale, d_rq=rq, d_rq_zp11=rq_zp, d_rq_div_zpm3=rq_div,
               d_brq=brq, d_scales_mid=sc_mid, d_rq_mid_zp5=rq_mid)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_golden.npz")
    np.savez_compressed(path, **{k: (v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v))
                                 for k, v in out.items()})
    print("wrote", path, os.path.getsize(path), "bytes;", "torch", torch.__version__)


if __name__ == "__main__":
    main()
