"""Synthetic 24-layer decoder projection stack (benchmark configuration 4), shared by the CPU oracle run and the
GPU run.  Hidden 1024, intermediate 3584; per layer q/k/v/o (1024x1024) chained, then gate/up (1024x3584), SiLU * up,
down (3584x1024); every projection is Cast(BF16 -> E5M2) -> MatMul(E5M2) -> Cast(E5M2 -> BF16) with per-tensor
power-of-two scales; BF16 residual adds; RMSNorm in FP32 with BF16 in/out (src/kernel/common/qwen_rms_norm.cc:71-95,
weight offset 1).  run_stack drives the stack with a `project` callback and the neighbours (QwenRmsNorm, Add, SiLU,
Mul) computed by the CPU oracle — the restatement of the reference's Common kernels pinned in
tests/test_oracle_decoder_ops.py; tests/test_gpu_decoder_step.py runs the whole step on the GPU against it."""
from __future__ import annotations

import numpy as np

HIDDEN, INTER, LAYERS = 1024, 3584, 24
ACT_SCALE = 2.0 ** -9   # exporter rule for amax 96: 2^ceil(log2(96 / 57344))
OUT_SCALE = 2.0 ** -9
EPS = np.float32(1e-6)
PROJ = [("q", HIDDEN, HIDDEN), ("k", HIDDEN, HIDDEN), ("v", HIDDEN, HIDDEN), ("o", HIDDEN, HIDDEN),
        ("gate", HIDDEN, INTER), ("up", HIDDEN, INTER), ("down", INTER, HIDDEN)]


def to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> BF16 bits, round to nearest even (finite inputs)."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def make_weights(encode_e5m2, seed=0xFEA70004, layers=LAYERS):
    """encode_e5m2(float32 array) -> E5M2 codes.  Returns per layer: codes + power-of-two scale per projection and
    the two RMSNorm weight vectors (BF16 bits)."""
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(layers):
        layer = {}
        for name, k, n in PROJ:
            w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
            scale = float(2.0 ** np.ceil(np.log2(np.abs(w).max() / 57344.0)))
            layer[name] = (encode_e5m2(w / np.float32(scale)), scale)
        layer["g1"] = to_bf16((rng.standard_normal(HIDDEN) * 0.1).astype(np.float32))
        layer["g2"] = to_bf16((rng.standard_normal(HIDDEN) * 0.1).astype(np.float32))
        out.append(layer)
    return out


def rmsnorm(x_bits, g_bits):
    """QwenRmsNorm node: the pinned restatement of the reference's Common kernel (weight offset 1, BF16 in / out)."""
    import oracle as O
    return O.qwen_rms_norm(O.BF16, x_bits, O.BF16, g_bits, 1.0, float(EPS), O.BF16)


def add(a_bits, b_bits):
    import oracle as O
    return O.binary(0, O.BF16, a_bits, b_bits)


def silu_mul(g_bits, u_bits):
    import oracle as O
    return O.binary(1, O.BF16, O.silu(O.BF16, g_bits), u_bits)   # SiLU node then Mul node, BF16 out each


def run_stack(project, weights, x_bits, trace=None, states=None):
    """project(h_bits [M,K] uint16, (codes, scale)) -> BF16 bits [M,N].  Returns the final hidden state (BF16 bits).
    `states`, when a list, receives the hidden state in front of every layer and the final one."""
    x = x_bits
    for layer in weights:
        if states is not None:
            states.append(x)
        h = rmsnorm(x, layer["g1"])
        t = h
        for name in ("q", "k", "v", "o"):
            if trace is not None:
                trace.append((name, t))
            t = project(t, layer[name])
        x = add(x, t)
        h = rmsnorm(x, layer["g2"])
        if trace is not None:
            trace.append(("gate", h))
            trace.append(("up", h))
        a = silu_mul(project(h, layer["gate"]), project(h, layer["up"]))
        if trace is not None:
            trace.append(("down", a))
        x = add(x, project(a, layer["down"]))
    if states is not None:
        states.append(x)
    return x
