"""One decode / prefill-chunk step of a projection stack, issued as C-ABI calls on one stream.

The layer is the one the synthetic 24-layer configuration uses (hidden H, intermediate I, BF16 residual stream, FP8
projections wrapped in Cast nodes, QwenRmsNorm with weight offset 1, SiLU * Mul between gate / up and down):

    h = QwenRmsNorm(x, g1);  t = o(v(k(q(h))));  x = Add(x, t)
    h = QwenRmsNorm(x, g2);  a = Mul(SiLU(gate(h)), up(h));  x = Add(x, down(a))

`fused=True` issues six launches per layer through fth_b200_fp8_linear_fused — norm + q, k, v, o + residual,
norm + gate | up + SiLU * Mul (one launch, two weights), down + residual — and every launch whose output feeds the next
projection directly also stores the FP8 codes that projection's Cast would make of it (out_codes), so that k, v, o and
down read 8-bit activations and run no Cast of their own; `fused=False` issues every node's own kernel
(twelve launches per layer: fth_b200_qwen_rms_norm, the Cast -> MatMul -> Cast projections, fth_b200_binary,
fth_b200_silu_mul).  Both give the same bytes.  Everything stays on the device; the caller may capture `run` in a CUDA
graph.  torch supplies the device buffers only.
"""
from __future__ import annotations

import ctypes as C

import infer_b200 as B


class DecoderStep:
    def __init__(self, torch, layers, m, hidden, inter, act_scale, out_scale, fp8_dtype=None, epsilon=1e-6, fused=True):
        """layers: per layer a dict with device tensors q, k, v, o, gate, up, down (FP8 codes, [K,N]) + their scales
        ("q_scale", ...) and g1, g2 (BF16 bits as int16 tensors, [hidden])."""
        self.torch, self.layers, self.m, self.hidden, self.inter = torch, layers, m, hidden, inter
        self.act_scale, self.out_scale, self.eps, self.fused = act_scale, out_scale, epsilon, fused
        self.dtype = fp8_dtype or B.E5M2
        bf = dict(dtype=torch.int16, device="cuda")
        self.x = torch.zeros((m, hidden), **bf)          # residual stream (input and output of the step)
        self.h = torch.zeros((m, hidden), **bf)
        self.t = [torch.zeros((m, hidden), **bf) for _ in range(2)]
        self.x2 = torch.zeros((m, hidden), **bf)
        self.gate = torch.zeros((m, inter), **bf)
        self.up = torch.zeros((m, inter), **bf)
        self.act = torch.zeros((m, inter), **bf)
        codes = dict(dtype=torch.uint8, device="cuda")
        self.c = [torch.zeros((m, hidden), **codes) for _ in range(2)]   # FP8 codes of t[0] / t[1] for the next projection
        self.act_codes = torch.zeros((m, inter), **codes)
        self.keep = []
        self.calls = []
        self._build()

    # ---- descriptors -------------------------------------------------------------------------------------------------
    def _proj(self, a, w, w_scale, out, k, n, codes_in=False):
        """codes_in: `a` holds the FP8 codes of the activation already (a producer's out_codes)."""
        d = B.fp8_linear_desc(dtype=self.dtype, op=B.OP_MATMUL, m=self.m, k=k, n=n, a=a, w=w, out=out, a_scale=self.act_scale,
                              w_scale=w_scale, out_scale=self.out_scale, a_dtype=0 if codes_in else B.BF16, out_dtype=B.BF16,
                              weights_static=True)
        self.keep.append(B.linear_workspace(self.torch, d))
        return d

    def _plain(self, d):
        self.calls.append(("linear", d, None))

    def _fused(self, d, **kw):
        f = B.fp8_linear_fusion(**kw)
        rc = B.lib().fth_b200_fp8_linear_fused_supported(C.byref(d), C.byref(f))
        if rc != 0:
            raise B.B200Error(rc, "fth_b200_fp8_linear_fused_supported")
        self.calls.append(("fused", d, f))

    def _build(self):
        H, I, m = self.hidden, self.inter, self.m
        x, nxt = self.x, self.x2
        for layer in self.layers:
            if self.fused:
                cast = dict(out_codes_scale=self.act_scale)  # the Cast in front of the next projection, run by the producer
                self._fused(self._proj(x, layer["q"], layer["q_scale"], self.t[0], H, H), prologue=B.FUSE_RMS_NORM, norm_weight=layer["g1"],
                            norm_weight_offset=1.0, norm_epsilon=self.eps, out_codes=self.c[0], **cast)
                self._fused(self._proj(self.c[0], layer["k"], layer["k_scale"], self.t[1], H, H, codes_in=True), out_codes=self.c[1], **cast)
                self._fused(self._proj(self.c[1], layer["v"], layer["v_scale"], self.t[0], H, H, codes_in=True), out_codes=self.c[0], **cast)
                self._fused(self._proj(self.c[0], layer["o"], layer["o_scale"], nxt, H, H, codes_in=True), residual=x)
                x, nxt = nxt, x
                self._fused(self._proj(x, layer["gate"], layer["gate_scale"], self.gate, H, I), prologue=B.FUSE_RMS_NORM, norm_weight=layer["g2"],
                            norm_weight_offset=1.0, norm_epsilon=self.eps, w2=layer["up"], w2_scale=layer["up_scale"], n2=I,
                            epilogue=B.FUSE_OUT_SILU_MUL, out_codes=self.act_codes, **cast)
                self._fused(self._proj(self.act_codes, layer["down"], layer["down_scale"], nxt, I, H, codes_in=True), residual=x)
                x, nxt = nxt, x
            else:
                self.calls.append(("norm", (x, layer["g1"], self.h), None))
                self._plain(self._proj(self.h, layer["q"], layer["q_scale"], self.t[0], H, H))
                self._plain(self._proj(self.t[0], layer["k"], layer["k_scale"], self.t[1], H, H))
                self._plain(self._proj(self.t[1], layer["v"], layer["v_scale"], self.t[0], H, H))
                self._plain(self._proj(self.t[0], layer["o"], layer["o_scale"], self.t[1], H, H))
                self.calls.append(("add", (x, self.t[1], nxt, m * H), None))
                x, nxt = nxt, x
                self.calls.append(("norm", (x, layer["g2"], self.h), None))
                self._plain(self._proj(self.h, layer["gate"], layer["gate_scale"], self.gate, H, I))
                self._plain(self._proj(self.h, layer["up"], layer["up_scale"], self.up, H, I))
                self.calls.append(("silu_mul", (self.gate, self.up, self.act, m * I), None))
                self._plain(self._proj(self.act, layer["down"], layer["down_scale"], self.t[0], I, H))
                self.calls.append(("add", (x, self.t[0], nxt, m * H), None))
                x, nxt = nxt, x
        self.result = x  # the buffer that holds the final hidden state after run()

    # ---- one step ----------------------------------------------------------------------------------------------------
    def run(self, stream=None):
        """Issues the whole step on `stream` (default: torch's current stream).  self.x holds the input, self.result
        the output (an even number of residual updates brings it back to self.x)."""
        lib = B.lib()
        s = stream or B.current_stream()
        for kind, d, f in self.calls:
            if kind == "linear":
                rc = lib.fth_b200_fp8_linear(C.byref(d), s)
            elif kind == "fused":
                rc = lib.fth_b200_fp8_linear_fused(C.byref(d), C.byref(f), s)
            elif kind == "norm":
                x, g, out = d
                rc = lib.fth_b200_qwen_rms_norm(C.c_int32(B.BF16), C.c_void_p(x.data_ptr()), C.c_int32(B.BF16), C.c_void_p(g.data_ptr()), C.c_float(1.0),
                                                C.c_float(self.eps), C.c_int32(B.BF16), C.c_void_p(out.data_ptr()), C.c_int64(self.m), C.c_int64(self.hidden), s)
            elif kind == "add":
                a, b, out, count = d
                rc = lib.fth_b200_binary(C.c_int32(B.BINARY_ADD), C.c_int32(B.BF16), C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()),
                                         C.c_void_p(out.data_ptr()), C.c_int64(count), C.c_int64(0), s)
            else:
                g, u, out, count = d
                rc = lib.fth_b200_silu_mul(C.c_int32(B.BF16), C.c_void_p(g.data_ptr()), C.c_void_p(u.data_ptr()), C.c_void_p(out.data_ptr()),
                                           C.c_int64(count), s)
            if rc != 0:
                raise B.B200Error(rc, f"decoder step ({kind})")

    @property
    def launches(self):
        return len(self.calls)


def _main():
    """Runs the synthetic stack a few times with random weights and prints the time per step (CUDA events), e.g. as the
    workload of a profiler capture: python -m infer_b200.decoder_step --m 16 --layers 4"""
    import argparse

    import torch

    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--inter", type=int, default=3584)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--nodes", action="store_true", help="every node as its own launch instead of the fused calls")
    args = ap.parse_args()
    H, I = args.hidden, args.inter
    shapes = {"q": (H, H), "k": (H, H), "v": (H, H), "o": (H, H), "gate": (H, I), "up": (H, I), "down": (I, H)}
    gen = torch.Generator(device="cuda").manual_seed(7)
    weights = []
    for _ in range(args.layers):
        layer = {}
        for name, (k, n) in shapes.items():
            layer[name] = torch.randint(0, 120, (k, n), dtype=torch.uint8, device="cuda", generator=gen)
            layer[name + "_scale"] = 2.0 ** -20
        for g in ("g1", "g2"):
            layer[g] = (torch.randn(H, device="cuda", generator=gen) * 0.1).to(torch.bfloat16).view(torch.int16)
        weights.append(layer)
    step = DecoderStep(torch, weights, args.m, H, I, 2.0 ** -9, 2.0 ** -9, fused=not args.nodes)
    step.x.copy_(torch.randn((args.m, H), device="cuda", generator=gen).to(torch.bfloat16).view(torch.int16))
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    step.run()
    torch.cuda.synchronize()
    begin.record()
    for _ in range(args.steps):
        step.run()
    end.record()
    torch.cuda.synchronize()
    print(f"m={args.m} layers={args.layers} launches/step={step.launches} {begin.elapsed_time(end) / args.steps * 1e3:.1f} us/step "
          f"(stream launches, no graph) status={B.device_status()}")


if __name__ == "__main__":
    _main()
