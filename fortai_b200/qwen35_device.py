"""The device pipeline of the reference's model object, restated over the C ABI mirror.

Follows qwen35_cpu_model_t with `cuda_device_pipeline` on
(src/models/qwen35/fortai_qwen35_cpu.f90): enable_cuda :287-384 (one context, every Q8_0
matrix uploaded, one layer object per layer borrowing the handles, five hidden-size fp32
buffers, the logits buffer and the norm weights on the device), forward :591-710
(embedding row on the device, position word, per layer copy -> rms_norm -> layer object ->
add -> copy -> rms_norm -> FFN -> add :713-747 and :764-800, output norm + lm_head :749-762,
one download of the logits), and the optional CUDA graph: captured on the first call with
position > 0 and relaunched afterwards :622-632, 694-700.

Every projection inside is the Q8_0 GEMV of this package; nothing here computes on the
host.  Weights come from `synthetic_model` (no GGUF model file exists in this image) or
from any dictionary of the same shape, e.g. filled from gguf_runtime tensors.
"""
from __future__ import annotations

import numpy as np

from . import backend_cuda as b

FORTAI_INVALID = b.FORTAI_INVALID


def synthetic_model(make_weights, hidden=256, inner=512, vocabulary=1024, layer_count=4,
                    attention_interval=4, max_context=32, seed=0, sigma=0.05):
    """Random-init weights with the layer pattern of Qwen3.5 (three gated-delta-net layers,
    then one attention layer).  `make_weights(rows, width, seed, sigma)` returns GGUF Q8_0
    bytes (tests pass the oracle's generator; the bench passes a device-side one)."""
    rng = np.random.default_rng(seed)
    heads, kv_heads, head_size = max(2, hidden // 128), max(1, hidden // 256), 64
    key_heads, value_heads, state = max(1, hidden // 256), max(2, hidden // 128), 64
    norm = lambda n: (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    counter = [seed * 1000 + 1]

    def q8(rows, width):
        counter[0] += 1
        return make_weights(rows, width, counter[0], sigma)

    spec = dict(hidden=hidden, inner=inner, vocabulary=vocabulary, max_context=max_context,
                epsilon=1e-6, token_embedding=q8(vocabulary, hidden), output=q8(vocabulary, hidden),
                output_norm=norm(hidden), layers=[])
    for index in range(layer_count):
        recurrent = (index + 1) % attention_interval != 0
        layer = dict(recurrent=recurrent, attn_norm=norm(hidden), post_norm=norm(hidden),
                     ffn_gate=q8(inner, hidden), ffn_up=q8(inner, hidden), ffn_down=q8(hidden, inner))
        if recurrent:
            conv_size = 2 * state * key_heads + value_heads * state
            value_inner = value_heads * state
            layer["mixer"] = dict(
                qkv=q8(conv_size, hidden), gate=q8(value_inner, hidden),
                alpha=q8(value_heads, hidden), beta=q8(value_heads, hidden),
                out=q8(hidden, value_inner), conv_kernel=4, conv_size=conv_size,
                conv_weights=(rng.standard_normal((conv_size, 4)) * 0.5).astype(np.float32),
                ssm_a=-np.exp(rng.standard_normal(value_heads)).astype(np.float32),
                ssm_dt=rng.standard_normal(value_heads).astype(np.float32), ssm_norm=norm(state),
                state_size=state, key_heads=key_heads, value_heads=value_heads, head_size=state,
                inner_size=value_inner)
        else:
            layer["mixer"] = dict(
                q=q8(heads * 2 * head_size, hidden), k=q8(kv_heads * head_size, hidden),
                v=q8(kv_heads * head_size, hidden), out=q8(hidden, heads * head_size),
                q_norm=norm(head_size), k_norm=norm(head_size), heads=heads, kv_heads=kv_heads,
                head_size=head_size, value_size=head_size, rope_dimension=head_size // 2,
                rope_base=1.0e7)
        spec["layers"].append(layer)
    return spec


class qwen35_device_model_t:
    def __init__(self):
        self.cuda = None
        self.spec = None
        self.cuda_graph_enabled = False
        self.cuda_graph_ready = False
        self.fused = False
        self._weights = []
        self._layers = []
        self._buffers = []

    # -- enable_cuda + setup_cuda_device_pipeline
    def open(self, spec, device=0, cuda_graph=False, fused=False) -> b.status_t:
        """`fused`: use the residual-stream entry points (norm and add inside the GEMVs)
        instead of the reference's copy / rms_norm / add calls around every layer half."""
        self.close()
        stat = b.status_t()
        self.cuda = b.cuda_q8_context_t()
        stat = self.cuda.create(device)
        if not stat.is_ok():
            return stat
        self.spec, self.cuda_graph_enabled, self.fused = spec, cuda_graph, fused
        hidden, vocabulary = spec["hidden"], spec["vocabulary"]

        def upload(host, rows, width):
            w = b.cuda_q8_weights_t()
            s = w.upload(self.cuda, host, host.size, rows, width)
            if not s.is_ok():
                raise RuntimeError(s.message + ": " + s.detail)
            self._weights.append(w)
            return w

        def device_floats(values):
            ptr = self.buffer(4 * values.size)
            s = self.cuda.upload(ptr, np.ascontiguousarray(values, np.float32))
            if not s.is_ok():
                raise RuntimeError(s.message)
            return ptr

        try:
            self.token_embedding = upload(spec["token_embedding"], vocabulary, hidden)
            self.output = upload(spec["output"], vocabulary, hidden)
            self.cuda_output_norm = device_floats(spec["output_norm"])
            for layer in spec["layers"]:
                entry = dict(recurrent=layer["recurrent"],
                             attn_norm=device_floats(layer["attn_norm"]),
                             post_norm=device_floats(layer["post_norm"]),
                             ffn_gate=upload(layer["ffn_gate"], spec["inner"], hidden),
                             ffn_up=upload(layer["ffn_up"], spec["inner"], hidden),
                             ffn_down=upload(layer["ffn_down"], hidden, spec["inner"]))
                m = layer["mixer"]
                if layer["recurrent"]:
                    obj = b.cuda_qwen35_recurrent_t()
                    s = obj.create(self.cuda, upload(m["qkv"], m["conv_size"], hidden),
                                   upload(m["gate"], m["inner_size"], hidden),
                                   upload(m["alpha"], m["value_heads"], hidden),
                                   upload(m["beta"], m["value_heads"], hidden),
                                   upload(m["out"], hidden, m["inner_size"]), m["conv_weights"],
                                   m["conv_size"], m["conv_kernel"], m["ssm_a"], m["ssm_dt"],
                                   m["ssm_norm"], m["state_size"], m["key_heads"], m["value_heads"],
                                   m["head_size"], m["inner_size"], spec["epsilon"])
                else:
                    obj = b.cuda_qwen35_attention_t()
                    s = obj.create(self.cuda, upload(m["q"], m["heads"] * 2 * m["head_size"], hidden),
                                   upload(m["k"], m["kv_heads"] * m["head_size"], hidden),
                                   upload(m["v"], m["kv_heads"] * m["value_size"], hidden),
                                   upload(m["out"], hidden, m["heads"] * m["value_size"]),
                                   m["q_norm"], m["k_norm"], m["heads"], m["kv_heads"],
                                   m["head_size"], m["value_size"], spec["max_context"],
                                   m["rope_dimension"], m["rope_base"], spec["epsilon"])
                if not s.is_ok():
                    raise RuntimeError(s.message + ": " + s.detail)
                entry["mixer"] = obj
                self._layers.append(entry)
            self.cuda_x = self.buffer(4 * hidden)
            self.cuda_residual = self.buffer(4 * hidden)
            self.cuda_normalized = self.buffer(4 * hidden)
            self.cuda_hidden = self.buffer(4 * hidden)
            self.cuda_logits = self.buffer(4 * vocabulary)
        except RuntimeError as error:
            self.close()
            stat.set(b.FORTAI_UNSUPPORTED, "Qwen3.5 CUDA device pipeline setup failed", str(error))
        return stat

    def buffer(self, nbytes):
        ptr, stat = self.cuda.allocate_buffer(nbytes)
        if not stat.is_ok():
            raise RuntimeError(stat.message)
        self._buffers.append(ptr)
        return ptr

    def close(self):
        # layers before weights: the layer objects borrow the weight handles
        for entry in self._layers:
            entry["mixer"].destroy()
        for w in self._weights:
            w.destroy()
        if self.cuda is not None:
            for ptr in self._buffers:
                self.cuda.free_buffer(ptr)
            self.cuda.destroy()
        self.__init__()

    def reset(self) -> b.status_t:
        stat = b.status_t()
        for entry in self._layers:
            stat = entry["mixer"].reset()
            if not stat.is_ok():
                return stat
        return stat

    # -- forward
    def _mix_and_ffn(self, entry, position) -> b.status_t:
        c, hidden = self.cuda, self.spec["hidden"]
        eps = self.spec["epsilon"]
        if self.fused:
            if entry["recurrent"]:
                stat = entry["mixer"].step_device(self.cuda_x, hidden, entry["attn_norm"], eps)
            else:
                stat = entry["mixer"].step_device(self.cuda_x, hidden, position,
                                                  entry["attn_norm"], eps)
            if stat.is_ok():
                stat = b.cuda_q8_ffn_step_device(c, entry["ffn_gate"], entry["ffn_up"],
                                                 entry["ffn_down"], self.cuda_x, hidden,
                                                 entry["post_norm"], eps)
            return stat
        stat = b.cuda_qwen35_copy_device(c, self.cuda_x, self.cuda_residual, 4 * hidden)
        if stat.is_ok():
            stat = b.cuda_qwen35_rms_norm_device(c, self.cuda_x, entry["attn_norm"],
                                                 self.cuda_normalized, hidden, eps)
        if stat.is_ok():
            if entry["recurrent"]:
                stat = entry["mixer"].run_device(self.cuda_normalized, hidden, self.cuda_hidden,
                                                 hidden)
            else:
                stat = entry["mixer"].run_device(self.cuda_normalized, hidden, position,
                                                 self.cuda_hidden, hidden)
        if stat.is_ok():
            stat = b.cuda_qwen35_add_device(c, self.cuda_hidden, self.cuda_residual, self.cuda_x,
                                            hidden)
        if stat.is_ok():
            stat = b.cuda_qwen35_copy_device(c, self.cuda_x, self.cuda_residual, 4 * hidden)
        if stat.is_ok():
            stat = b.cuda_qwen35_rms_norm_device(c, self.cuda_x, entry["post_norm"],
                                                 self.cuda_normalized, hidden, eps)
        if stat.is_ok():
            stat = b.cuda_q8_ffn_device(c, entry["ffn_gate"], entry["ffn_up"], entry["ffn_down"],
                                        self.cuda_normalized, hidden, self.cuda_hidden, hidden)
        if stat.is_ok():
            stat = b.cuda_qwen35_add_device(c, self.cuda_hidden, self.cuda_residual, self.cuda_x,
                                            hidden)
        return stat

    def _output(self) -> b.status_t:
        hidden = self.spec["hidden"]
        if self.fused:
            return b.cuda_q8_matvec_norm_device_f32(self.cuda, self.output, self.cuda_x, hidden,
                                                    self.cuda_output_norm, self.spec["epsilon"],
                                                    self.cuda_logits, self.spec["vocabulary"])
        stat = b.cuda_qwen35_rms_norm_device(self.cuda, self.cuda_x, self.cuda_output_norm,
                                             self.cuda_normalized, hidden, self.spec["epsilon"])
        if stat.is_ok():
            stat = b.cuda_q8_matvec_device_f32(self.cuda, self.output, self.cuda_normalized, hidden,
                                               self.cuda_logits, self.spec["vocabulary"])
        return stat

    def forward(self, token_id: int, position: int):
        """One decode step; returns (logits, status)."""
        stat = b.status_t()
        if self.cuda is None:
            stat.set(FORTAI_INVALID, "Qwen3.5 CPU model is not open")
            return None, stat
        if token_id < 0 or token_id >= self.spec["vocabulary"]:
            stat.set(FORTAI_INVALID, "token id is outside the Qwen3.5 vocabulary")
            return None, stat
        if position < 0 or position >= self.spec["max_context"]:
            stat.set(FORTAI_INVALID, "Qwen3.5 position exceeds the CPU context")
            return None, stat
        stat = b.cuda_qwen35_embedding_device(self.cuda, self.token_embedding, token_id, self.cuda_x,
                                              self.spec["hidden"])
        if stat.is_ok():
            stat = self.cuda.set_position(position)
        if not stat.is_ok():
            return None, stat
        capture = False
        if self.cuda_graph_enabled:
            if self.cuda_graph_ready:
                stat = self.cuda.graph_launch()
            elif position > 0:
                stat = self.cuda.capture_begin()
                capture = True
            if not stat.is_ok():
                return None, stat
        if not (self.cuda_graph_enabled and self.cuda_graph_ready):
            for entry in self._layers:
                stat = self._mix_and_ffn(entry, position)
                if not stat.is_ok():
                    return None, stat
            stat = self._output()
            if not stat.is_ok():
                return None, stat
        if capture:
            stat = self.cuda.capture_end()
            if stat.is_ok():
                self.cuda_graph_ready = True
                stat = self.cuda.graph_launch()
            if not stat.is_ok():
                return None, stat
        return self.cuda.download_real(self.cuda_logits, self.spec["vocabulary"])
