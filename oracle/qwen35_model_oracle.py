"""CPU restatement of one decode step of the reference model (TEST INFRASTRUCTURE ONLY):
qwen35_cpu_forward on its CPU path, src/models/qwen35/fortai_qwen35_cpu.f90:591-710
(embedding row :618, per layer: rms_norm :1408-1432 -> recurrent or attention -> residual
add -> rms_norm -> FFN = matvec pair, silu product, matvec :673-679 -> residual add; output
norm and lm_head :706-709).  Built from the pinned Q8_0 oracle and the layer oracle; the
Fortran glue itself cannot be compiled here, so whole-model parity is UNPINNED.
"""
from __future__ import annotations

import numpy as np

from . import q8_oracle as o
from . import qwen35_layers_oracle as lo

f32 = np.float32


def rms_norm(x, weights, epsilon):
    total = float(np.sum(x.astype(np.float64) ** 2))
    mean = f32(total / x.size)
    inverse = f32(1.0) / np.sqrt(mean + f32(epsilon), dtype=f32)
    return ((x * inverse).astype(f32) * weights).astype(f32)


class Model:
    """`spec` is the dictionary produced by fortai_b200.qwen35_device.synthetic_model."""

    def __init__(self, spec):
        self.s = spec
        self.layers = []
        for layer in spec["layers"]:
            if layer["recurrent"]:
                r = layer["mixer"]
                mixer = lo.Recurrent(r["qkv"], r["gate"], r["alpha"], r["beta"], r["out"],
                                     spec["hidden"], r["conv_weights"], r["conv_kernel"], r["ssm_a"],
                                     r["ssm_dt"], r["ssm_norm"], r["state_size"], r["key_heads"],
                                     r["value_heads"], r["head_size"], f32(spec["epsilon"]))
            else:
                a = layer["mixer"]
                mixer = lo.Attention(a["q"], a["k"], a["v"], a["out"], spec["hidden"], a["q_norm"],
                                     a["k_norm"], a["heads"], a["kv_heads"], a["head_size"],
                                     a["value_size"], spec["max_context"], a["rope_dimension"],
                                     f32(a["rope_base"]), f32(spec["epsilon"]))
            self.layers.append(mixer)

    def forward(self, token_id, position):
        s = self.s
        hidden, inner = s["hidden"], s["inner"]
        x = o.dequantize_row(s["token_embedding"], token_id, hidden // 32)
        for layer, mixer in zip(s["layers"], self.layers):
            normalized = rms_norm(x, layer["attn_norm"], s["epsilon"])
            mixed = mixer.run(normalized) if layer["recurrent"] else mixer.run(normalized, position)
            x = (mixed + x).astype(f32)
            normalized = rms_norm(x, layer["post_norm"], s["epsilon"])
            x = (o.ffn(layer["ffn_gate"], layer["ffn_up"], layer["ffn_down"], inner, hidden, hidden,
                       normalized) + x).astype(f32)
        normalized = rms_norm(x, s["output_norm"], s["epsilon"])
        return o.matvec(s["output"], s["vocabulary"], hidden, normalized)[0]
