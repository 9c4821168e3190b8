"""Independent double-precision model of the Qwen sequence attention forward, used to check
gradients by central differences the way the reference's own test does
(src/llm/layers/qwen_attention_test.cc:22-100, 230-301): every bf16 rounding is replaced by
"add the rounding error recorded on the unperturbed inputs", so a cast has derivative one and
the finite difference never crosses a quantisation step."""
import math

import numpy as np

import oracle


def bf16(x: float) -> float:
    return float(oracle.round_bf16(np.array([x], np.float32))[0])


class DoubleModel:
    def __init__(self, t, hq, hkv, d, rotary, eps, theta, rnd):
        self.t, self.hq, self.hkv, self.d = t, hq, hkv, d
        self.rotary, self.eps, self.theta, self.rnd = rotary, eps, theta, rnd
        self.errors = []
        self.recording = False
        self.index = 0

    def _round(self, value):
        if not self.rnd:
            return value
        if self.recording:
            self.errors.append(bf16(value) - value)
        value += self.errors[self.index]
        self.index += 1
        return value

    def _prepare(self, x, w, heads, stride):
        t, d, rot = self.t, self.d, self.rotary
        out = [0.0] * (t * heads * d)
        for row in range(t):
            for h in range(heads):
                base, o = (row * heads + h) * stride, (row * heads + h) * d
                ss = sum(x[base + c] ** 2 for c in range(d))
                inv = 1.0 / math.sqrt(ss / d + self.eps)
                for c in range(d):
                    out[o + c] = self._round(x[base + c] * inv * (1 + w[c]))
                for c in range(rot // 2):
                    partner = c + rot // 2
                    a = row * self.theta ** (-2.0 * c / rot)
                    first, second = out[o + c], out[o + partner]
                    cosine, sine = self._round(math.cos(a)), self._round(math.sin(a))
                    fc, ss2 = self._round(first * cosine), self._round(second * sine)
                    sc, fs = self._round(second * cosine), self._round(first * sine)
                    out[o + c] = self._round(fc - ss2)
                    out[o + partner] = self._round(sc + fs)
        return out

    def forward(self, qg, k, v, qw, kw, record=False):
        """Flat python lists in, flat list [T*Hq*D] out."""
        self.recording, self.index = record, 0
        if record:
            self.errors = []
        t, hq, hkv, d = self.t, self.hq, self.hkv, self.d
        query = self._prepare(qg, qw, hq, 2 * d)
        key = self._prepare(k, kw, hkv, d)
        out = [0.0] * (t * hq * d)
        for row in range(t):
            for h in range(hq):
                kv = h // (hq // hkv)
                prob = [sum(query[(row * hq + h) * d + c] * key[(s * hkv + kv) * d + c]
                            for c in range(d)) / math.sqrt(d) for s in range(row + 1)]
                m = max(prob)
                prob = [math.exp(x - m) for x in prob]
                z = sum(prob)
                for c in range(d):
                    core = sum(prob[s] / z * v[(s * hkv + kv) * d + c] for s in range(row + 1))
                    rc = self._round(core)
                    gate = self._round(1 / (1 + math.exp(-qg[((row * hq + h) * 2 + 1) * d + c])))
                    out[(row * hq + h) * d + c] = self._round(rc * gate)
        return out

    def gradients(self, inputs, upstream, step=1e-5):
        """Central differences of sum(forward * upstream) w.r.t. every entry of the five inputs
        (qg, k, v, qw, kw), rounding errors frozen at the unperturbed point."""
        inputs = [list(map(float, x)) for x in inputs]
        self.forward(*inputs, record=True)

        def loss():
            y = self.forward(*inputs)
            return sum(a * b for a, b in zip(y, upstream))

        grads = []
        for which in range(len(inputs)):
            g = []
            for i in range(len(inputs[which])):
                original = inputs[which][i]
                inputs[which][i] = original + step
                plus = loss()
                inputs[which][i] = original - step
                minus = loss()
                inputs[which][i] = original
                g.append((plus - minus) / (2 * step))
            grads.append(np.array(g))
        return grads


def wave(n, phase):
    """The reference test's input generator: bf16(0.8 sin(phase + 0.29 i))."""
    return oracle.round_bf16((0.8 * np.sin(phase + 0.29 * np.arange(n))).astype(np.float32)).astype(np.float64)
