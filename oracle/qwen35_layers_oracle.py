"""CPU restatement of the reference's recurrent (gated-delta-net) and attention layers.
TEST INFRASTRUCTURE ONLY - nothing in the shipped package imports this module.

What is restated, and from where (paths inside the reference project):
  forward_recurrent      src/models/qwen35/fortai_qwen35_cpu.f90:801-918
  fortai_gdn_step        src/backend/cpu/fortai_q8_dot.c:355-445 (one head, one token)
  forward_attention      src/models/qwen35/fortai_qwen35_cpu.f90:978-1035
  normalize_slice        :1434-1453   (sum of squares in float64, RMS in float32)
  l2_normalize_slice     :1455-1471
  apply_rope             :1473-1497   (NeoX half-vector pairs)
  sigmoid / softplus     :1506-1526
  rms_slice              :1528-1539
  KV cache in binary16   :1584-1604

Parity pin: `gdn_step` is checked against the reference's compiled C function
(oracle/_ref) and against the known answer of test/test_fortai_smoke.f90:268-282; the
Q8_0 projections go through the pinned matvec oracle.  The Fortran glue around them
cannot be compiled in this image (no Fortran compiler), so for that glue the parity is
UNPINNED: it is a careful restatement, checked only for self-consistency.
"""
from __future__ import annotations

import numpy as np

from . import q8_oracle as o

f32 = np.float32


def sigmoid(v):
    v = f32(v)
    if v >= 0:
        return f32(1.0) / (f32(1.0) + np.exp(-v, dtype=f32))
    e = np.exp(v, dtype=f32)
    return e / (f32(1.0) + e)


def softplus(v):
    v = f32(v)
    if v > 20:
        return v
    if v < -20:
        return np.exp(v, dtype=f32)
    return np.log(f32(1.0) + np.exp(v, dtype=f32), dtype=f32)


def silu(values):
    """fortai_silu for checking purposes: x / (1 + exp(-x)) in float32 (the reference's
    AVX2 path approximates exp to 2e-7 relative; tests allow for that)."""
    x = values.astype(f32)
    return (x / (f32(1.0) + np.exp(-x, dtype=f32))).astype(f32)


def gdn_step(state, key, value, query, decay, beta, output_scale):
    """One head, one token; `state` is head_size x head_size, updated in place."""
    hs = key.size
    out = np.zeros(hs, f32)
    for row in range(hs):
        state[row] = (state[row] * f32(decay)).astype(f32)
        dot = f32(np.dot(state[row].astype(f32), key.astype(f32)))
        delta = f32((f32(value[row]) - dot) * f32(beta))
        state[row] = (state[row] + delta * key).astype(f32)
        out[row] = f32(np.dot(state[row], query)) * f32(output_scale)
    return out


def l2_normalize(values, epsilon):
    total = float(np.sum(values.astype(np.float64) ** 2))
    inverse = f32(1.0) / max(np.sqrt(f32(total)), f32(epsilon))
    return (values * inverse).astype(f32)


def normalize_slice(values, epsilon, weights):
    total = float(np.sum(values.astype(np.float64) ** 2))
    mean = f32(total / values.size)
    inverse = f32(1.0) / np.sqrt(mean + f32(epsilon), dtype=f32)
    return ((values * inverse).astype(f32) * weights).astype(f32)


def half_round(values):
    """float -> binary16 -> float, as the KV cache stores it."""
    return values.astype(np.float16).astype(f32)


class Recurrent:
    """State and weights of one gated-delta-net layer."""

    def __init__(self, qkv, gate, alpha, beta, out, hidden, conv_weights, conv_kernel, ssm_a,
                 ssm_dt, ssm_norm, state_size, key_heads, value_heads, head_size, epsilon):
        self.w = dict(qkv=qkv, gate=gate, alpha=alpha, beta=beta, out=out)
        self.hidden = hidden
        self.conv_size = 2 * state_size * key_heads + value_heads * head_size
        self.conv_kernel = conv_kernel
        self.conv_weights = conv_weights.astype(f32).reshape(self.conv_size, conv_kernel)
        self.ssm_a, self.ssm_dt, self.ssm_norm = ssm_a, ssm_dt, ssm_norm
        self.state_size, self.key_heads, self.value_heads = state_size, key_heads, value_heads
        self.head_size, self.epsilon = head_size, epsilon
        self.inner = value_heads * head_size
        self.reset()

    def reset(self):
        self.conv_state = np.zeros((self.conv_kernel - 1, self.conv_size), f32)
        self.gdn_state = np.zeros((self.value_heads, self.head_size, self.head_size), f32)

    def run(self, x):
        qkv = o.matvec(self.w["qkv"], self.conv_size, self.hidden, x)[0]
        gate = silu(o.matvec(self.w["gate"], self.inner, self.hidden, x)[0])
        alpha = o.matvec(self.w["alpha"], self.value_heads, self.hidden, x)[0]
        beta = o.matvec(self.w["beta"], self.value_heads, self.hidden, x)[0]
        # causal depthwise convolution over the last conv_kernel inputs, then SiLU
        acc = np.zeros(self.conv_size, f32)
        for slot in range(self.conv_kernel - 1):
            acc = (acc + self.conv_weights[:, slot] * self.conv_state[slot]).astype(f32)
        acc = (acc + self.conv_weights[:, self.conv_kernel - 1] * qkv).astype(f32)
        conv = silu(acc)
        self.conv_state[:-1] = self.conv_state[1:].copy()
        self.conv_state[-1] = qkv
        hs, kh = self.head_size, self.key_heads
        k_base = self.state_size * kh
        v_base = 2 * self.state_size * kh
        for head in range(kh):
            conv[head * hs:(head + 1) * hs] = l2_normalize(conv[head * hs:(head + 1) * hs],
                                                           self.epsilon)
            conv[k_base + head * hs:k_base + (head + 1) * hs] = l2_normalize(
                conv[k_base + head * hs:k_base + (head + 1) * hs], self.epsilon)
        attention = np.zeros(self.inner, f32)
        for head in range(self.value_heads):
            key_head = head // (self.value_heads // kh)
            b = sigmoid(beta[head])
            decay = np.exp(f32(self.ssm_a[head]) * softplus(alpha[head] + f32(self.ssm_dt[head])),
                           dtype=f32)
            key = conv[k_base + key_head * hs:k_base + (key_head + 1) * hs]
            query = conv[key_head * hs:(key_head + 1) * hs]
            value = conv[v_base + head * hs:v_base + (head + 1) * hs]
            out = gdn_step(self.gdn_state[head], key, value, query, decay, b,
                           f32(1.0) / np.sqrt(f32(hs)))
            total = float(np.sum(out.astype(np.float64) ** 2))
            norm = np.sqrt(f32(total / hs) + f32(self.epsilon), dtype=f32)
            attention[head * hs:(head + 1) * hs] = (out / norm * self.ssm_norm *
                                                    gate[head * hs:(head + 1) * hs]).astype(f32)
        rows = self.w["out"].size // ((self.inner // 32) * 34)
        return o.matvec(self.w["out"], rows, self.inner, attention)[0]


class Attention:
    """State and weights of one gated single-query attention layer."""

    def __init__(self, q, k, v, out, hidden, q_norm, k_norm, heads, kv_heads, head_size,
                 value_size, max_context, rope_dimension, rope_base, epsilon):
        self.w = dict(q=q, k=k, v=v, out=out)
        self.hidden, self.q_norm, self.k_norm = hidden, q_norm, k_norm
        self.heads, self.kv_heads, self.head_size = heads, kv_heads, head_size
        self.value_size, self.max_context = value_size, max_context
        self.rope_dimension, self.rope_base, self.epsilon = rope_dimension, rope_base, epsilon
        self.reset()

    def reset(self):
        self.key_cache = np.zeros((self.max_context, self.kv_heads, self.head_size), f32)
        self.value_cache = np.zeros((self.max_context, self.kv_heads, self.value_size), f32)

    def _rope(self, vector, position):
        half = self.rope_dimension // 2
        out = vector.copy()
        for i in range(half):
            angle = f32(position) / np.power(f32(self.rope_base),
                                             f32(2 * i) / f32(self.rope_dimension), dtype=f32)
            c, s = np.cos(angle, dtype=f32), np.sin(angle, dtype=f32)
            a, b = vector[i], vector[i + half]
            out[i] = a * c - b * s
            out[i + half] = a * s + b * c
        return out.astype(f32)

    def run(self, x, position):
        hs, vs = self.head_size, self.value_size
        qv, kv, vv = o.matvec_triplet(self.w["q"], self.w["k"], self.w["v"],
                                      (self.heads * 2 * hs, self.kv_heads * hs, self.kv_heads * vs),
                                      self.hidden, x)
        q = qv.copy()
        for head in range(self.heads):
            sl = slice(head * 2 * hs, head * 2 * hs + hs)
            q[sl] = normalize_slice(q[sl], self.epsilon, self.q_norm)
            if self.rope_dimension > 0:
                q[sl] = self._rope(q[sl], position)
        k = kv.copy()
        for head in range(self.kv_heads):
            sl = slice(head * hs, (head + 1) * hs)
            k[sl] = normalize_slice(k[sl], self.epsilon, self.k_norm)
            if self.rope_dimension > 0:
                k[sl] = self._rope(k[sl], position)
        self.key_cache[position] = half_round(k).reshape(self.kv_heads, hs)
        self.value_cache[position] = half_round(vv).reshape(self.kv_heads, vs)
        attention = np.zeros(self.heads * vs, f32)
        group = self.heads // self.kv_heads
        for head in range(self.heads):
            kvh = head // group
            query = q[head * 2 * hs:head * 2 * hs + hs]
            gate = q[head * 2 * hs + hs:head * 2 * hs + hs + vs]
            keys = self.key_cache[:position + 1, kvh]
            scores = (keys @ query).astype(f32) / np.sqrt(f32(hs))
            weights = np.exp(scores - scores.max(), dtype=f32)
            weights = (weights / weights.sum(dtype=f32)).astype(f32)
            mixed = (weights[:, None] * self.value_cache[:position + 1, kvh]).sum(axis=0,
                                                                                  dtype=f32)
            attention[head * vs:(head + 1) * vs] = mixed * np.array(
                [sigmoid(g) for g in gate], f32)
        rows = self.w["out"].size // ((self.heads * vs // 32) * 34)
        return o.matvec(self.w["out"], rows, self.heads * vs, attention)[0]
