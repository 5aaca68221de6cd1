"""Loading of the committed golden fixtures (outputs of the reference's own code, see
tests/golden/make_golden.py)."""
from __future__ import annotations

import ast
import os

import numpy as np
import torch

from socket_b200.synth import hypercube_protos, make_decode_inputs

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

OPS_CASES = ["tiny_rep4_f32", "tiny_rep4_bf16", "batch2_rep4_f32", "edge_short_ctx",
             "edge_no_base", "edge_masked", "rep1_mha", "rep8_gqa"]


class Case:
    pass


def _dtype(name: str):
    return {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16,
            "torch.float16": torch.float16}[name]


def load_ops_case(name: str) -> Case:
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    c = Case()
    c.name = name
    c.sink, c.window, c.M = int(z["sink"]), int(z["window"]), int(z["M"])
    c.meta = ast.literal_eval(str(z["meta"]))
    if "in_k" in z:
        dt = _dtype(str(z["in_dtype"]))
        c.dtype = dt

        def get(key):
            t = torch.from_numpy(z["in_" + key])
            return t.view(dt) if dt != torch.float32 else t
        c.planes, c.q, c.k, c.v = get("planes"), get("q"), get("k"), get("v")
        c.protos_T = torch.from_numpy(z["in_protos_T"])
    else:
        m = c.meta
        c.dtype = _dtype(m["dtype"])
        inp = make_decode_inputs(m["B"], m["H"], m["Hkv"], m["T"], D=m["D"], L=m["L"], P=m["P"],
                                 seed=m["seed"], dtype=c.dtype, plant_frac=m["plant_frac"])
        c.planes, c.q, c.k, c.v, c.protos_T = inp.planes, inp.q, inp.k, inp.v, inp.protos_T
        c.in_sha_k, c.in_sha_q = str(z["in_sha_k"]), str(z["in_sha_q"])
    c.codes_sha = str(z["codes_sha"])
    for key in ("codes", "q_probs", "scores", "sparse_list", "sparse_len", "out", "allowed"):
        setattr(c, key, torch.from_numpy(z[key]) if key in z else None)
    c.v_norm = torch.from_numpy(z["v_norm"]).view(torch.float16) if "v_norm" in z else None
    c.B, c.H, c.D = c.q.shape
    c.Hkv, c.T = c.k.shape[1], c.k.shape[2]
    c.L, c.P = c.planes.shape[0], c.planes.shape[1]
    c.rep = c.H // c.Hkv
    return c


def load_model_flow() -> Case:
    z = np.load(os.path.join(GOLDEN_DIR, "model_flow.npz"))
    c = Case()
    for key in z.files:
        v = z[key]
        if v.ndim == 0:
            setattr(c, key, int(v))
        elif key == "v_norm":
            setattr(c, key, torch.from_numpy(v).view(torch.float16))
        else:
            setattr(c, key, torch.from_numpy(v))
    return c
