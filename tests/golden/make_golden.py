"""Generate the golden fixtures in this directory from the reference itself.

Run once, in a container where the MindPipe reference checkout is present
(its path in ``MINDPIPE_REFERENCE``).  The script imports the
reference's own functions (nothing is copied), feeds them small seeded
inputs and stores inputs and outputs as ``.npz`` files.  The fixtures are
committed, so the tests never need the reference at run time.

    MINDPIPE_REFERENCE=<path to the reference checkout> python tests/golden/make_golden.py
"""
from __future__ import annotations

import importlib
import os
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

if "MINDPIPE_REFERENCE" not in os.environ:
    sys.exit("set MINDPIPE_REFERENCE to a checkout of the reference project")
REF = Path(os.environ["MINDPIPE_REFERENCE"])
OUT = Path(__file__).resolve().parent
sys.dont_write_bytecode = True
for sub in ("", "algorithm/quantization/ptq/awq/source", "algorithm/quantization/ptq/smoothquant/source",
            "algorithm/quantization/ptq/omniquant/source",
            "algorithm/quantization/ptq/gptq/source", "algorithm/quantization/qat/flatquant/source",
            "scripts/repro"):
    sys.path.insert(0, str(REF / sub))


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def np16(t):
    return t.detach().cpu().numpy()


def main():
    from awq.quantize.quantizer import pseudo_quantize_tensor
    from smoothquant.fake_quant import (SmoothQuantLinear, SmoothQuantPackedMoeExperts,
                                        quantize_activation_per_token_absmax,
                                        quantize_weight_per_channel_absmax)
    from algorithm.quantization.exporters.vllm import pack_int4_for_vllm
    deq = importlib.import_module("evaluate_real_quant_export_dequant")
    exp8 = importlib.import_module("export_fp16_to_ascend_w8a8_dynamic_probe")

    # ---- W4 asymmetric g128 (and the ragged-K fallback to one group per row) ----
    w = (torch.randn(24, 384, generator=gen(1)) * 0.02).half()
    wdq, s, z = pseudo_quantize_tensor(w, n_bit=4, zero_point=True, q_group_size=128, get_scale_zp=True)
    w_r = (torch.randn(8, 200, generator=gen(2)) * 0.02).half()
    wdq_r, s_r, z_r = pseudo_quantize_tensor(w_r, n_bit=4, zero_point=True, q_group_size=128, get_scale_zp=True)
    w_c = torch.zeros(4, 128).half()                       # constant group: exercises the 1e-5 clamp
    w_c[1] = 0.5
    w_c[2, :64] = -0.25
    wdq_c, s_c, z_c = pseudo_quantize_tensor(w_c, n_bit=4, zero_point=True, q_group_size=128, get_scale_zp=True)
    x = torch.randn(5, 384, generator=gen(3)).half()
    y = torch.nn.functional.linear(x, wdq)
    np.savez_compressed(OUT / "w4a16_small.npz", w=np16(w), wdq=np16(wdq), scales=np16(s), zeros=np16(z),
                        w_ragged=np16(w_r), wdq_ragged=np16(wdq_r), scales_ragged=np16(s_r), zeros_ragged=np16(z_r),
                        w_const=np16(w_c), wdq_const=np16(wdq_c), scales_const=np16(s_c), zeros_const=np16(z_c),
                        x=np16(x), y=np16(y))

    # ---- int4 pack / unpack / dequant of the exported (symmetric) format ----
    kat = torch.tensor([[-8, -7, -1, 0, 1, 6, 7, -3, 4, 2]], dtype=torch.int8)   # the reference test's vector
    kat_packed = pack_int4_for_vllm(kat)
    q = torch.randint(-8, 8, (6, 40), generator=gen(4), dtype=torch.int8)
    q_packed = pack_int4_for_vllm(q)
    sc = (torch.rand(6, 5, generator=gen(5)) * 0.01 + 0.001).half()
    q_dq = deq._dequantize_weight(packed=q_packed, scale=sc, weight_shape=torch.tensor([6, 40]))
    q_un = deq._unpack_int4(q_packed, (6, 40))
    np.savez_compressed(OUT / "int4_pack.npz", kat=np16(kat), kat_packed=np16(kat_packed), q=np16(q),
                        q_packed=np16(q_packed), q_unpacked=np16(q_un), scale=np16(sc), q_dequant_f32=np16(q_dq))

    # ---- GPTQ real-quant artifact (the reference test's recipe, larger) ----
    GPTQ = importlib.import_module("gptq").GPTQ
    Quantizer = importlib.import_module("quant").Quantizer
    torch.manual_seed(0)
    lin = torch.nn.Linear(64, 16, bias=False)
    g = GPTQ(lin)
    qz = Quantizer()
    qz.configure(4, perchannel=True, sym=True, mse=False)
    g.quantizer = qz
    inp = torch.randn(2, 32, 64)
    g.add_batch(inp, lin(inp))
    res = g.fasterquant(blocksize=16, percdamp=0.01, groupsize=32, return_real_quant=True)
    int_w = res["int_weight"].to(torch.int8)
    np.savez_compressed(OUT / "gptq_artifact.npz", int_weight=np16(int_w), scale=np16(res["scale"]),
                        packed=np16(pack_int4_for_vllm(int_w)), fake_weight=np16(lin.weight.detach().float()))

    # ---- W8A8 pieces ----
    xa = torch.randn(7, 256, generator=gen(6)).half()
    xa[:, [3, 77]] *= 20
    xa[5] = 0                                           # all-zero token: the 1e-5 clamp
    xq = quantize_activation_per_token_absmax(xa)
    w8 = (torch.randn(16, 256, generator=gen(7)) * 0.02).half()
    w8q = quantize_weight_per_channel_absmax(w8)
    e_q, e_s, e_o = exp8.quantize_weight_per_channel(w8)
    lin8 = torch.nn.Linear(256, 16, bias=True).half()
    with torch.no_grad():
        lin8.weight.copy_(w8)
        lin8.bias.copy_((torch.randn(16, generator=gen(8)) * 0.1).half())
    m_plain = SmoothQuantLinear.from_float(lin8)
    m_oq = SmoothQuantLinear.from_float(lin8, quantize_output=True)
    np.savez_compressed(OUT / "w8a8_small.npz", x=np16(xa), x_fake=np16(xq), w=np16(w8), w_fake=np16(w8q),
                        exp_q=np16(e_q), exp_scale=np16(e_s), exp_offset=np16(e_o), bias=np16(lin8.bias),
                        y=np16(m_plain(xa)), y_outq=np16(m_oq(xa)))

    # ---- OmniQuant-style asymmetric per-token activations / per-channel weights ----
    oq = importlib.import_module("omniquant.int_linear")
    lin_o = torch.nn.Linear(256, 16, bias=True).half()
    with torch.no_grad():
        lin_o.weight.copy_(w8)
        lin_o.bias.copy_(lin8.bias)
    act_p = {"n_bits": 8, "per_channel_axes": [], "symmetric": False, "dynamic_method": "per_token"}
    w_p = {"n_bits": 8, "per_channel_axes": [0], "symmetric": False, "dynamic_method": "per_channel",
           "group_size": None, "lwc": False, "disable_zero_point": False}
    ql = oq.QuantLinear(lin_o, weight_quant_params=w_p, act_quant_params=act_p)
    ql.set_quant_state(weight_quant=True, act_quant=True)
    with torch.no_grad():
        xo = xa.clone()
        xo[5] = xa[4] + 0.25                                # no all-zero row: keep the ranges ordinary
        y_o = ql(xo)
        x_fake_o = ql.act_quantizer(xo.clone())
        x_scale_o, x_zp_o = ql.act_quantizer.scale.clone(), ql.act_quantizer.round_zero_point.clone()
        w_fake_o = ql.weight_quantizer(w8.clone())
        w_scale_o, w_zp_o = ql.weight_quantizer.scale.clone(), ql.weight_quantizer.round_zero_point.clone()
    np.savez_compressed(OUT / "omniquant_small.npz", x=np16(xo), w=np16(w8), bias=np16(lin8.bias), y=np16(y_o),
                        x_fake=np16(x_fake_o), x_scale=np16(x_scale_o), x_zp=np16(x_zp_o),
                        w_fake=np16(w_fake_o), w_scale=np16(w_scale_o), w_zp=np16(w_zp_o))

    # ---- MoE ----
    E, H, I, T, K = 4, 128, 192, 40, 2
    gu = (torch.randn(E, 2 * I, H, generator=gen(9)) * 0.05).half()
    dn = (torch.randn(E, H, I, generator=gen(10)) * 0.05).half()
    hs = torch.randn(T, H, generator=gen(11)).half()
    logits = torch.randn(T, E, generator=gen(12))
    logits[:, 3] -= 100.0                               # expert 3 is never hit
    try:
        # flatquant.utils imports three names from `accelerate` (absent offline) at module
        # import time; the router method below never touches them, so stand-ins suffice.
        import types
        if "accelerate" not in sys.modules:
            acc = types.ModuleType("accelerate")
            acc.dispatch_model = acc.infer_auto_device_map = None
            acc_utils = types.ModuleType("accelerate.utils")
            acc_utils.get_balanced_memory = None
            acc.utils = acc_utils
            sys.modules["accelerate"], sys.modules["accelerate.utils"] = acc, acc_utils
        mu = importlib.import_module("flatquant.model_tools.mixtral_utils")
        stub = SimpleNamespace(_ori_mode=True, _eval_mode=False, gate=lambda h: logits, top_k=K)
        _, rw, sel = mu.FlatQuantMixtralSparseMoeBlock._route(stub, hs)
        router_src = "reference:_route"
    except Exception as err:                            # pragma: no cover
        raise SystemExit(f"router import failed: {err!r}")
    rw16 = rw.to(hs.dtype)
    src = SimpleNamespace(gate_up_proj=gu, down_proj=dn, act_fn=torch.nn.SiLU())
    moe = SmoothQuantPackedMoeExperts.from_float(src)
    out = moe(hs, sel, rw16)
    np.savez_compressed(OUT / "moe_small.npz", gate_up=np16(gu), down=np16(dn), hidden=np16(hs),
                        logits=np16(logits), top_k_index=np16(sel), top_k_weights=np16(rw16),
                        top_k_weights_f32=np16(rw), gate_up_fake=np16(moe.gate_up_proj),
                        down_fake=np16(moe.down_proj), out=np16(out))
    print("router source:", router_src)
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
