"""Independent double-precision model of the SequenceDeltaNetLayer forward with frozen rounding
offsets, for gradient checks by central differences as the reference's own test does
(src/llm/layers/sequence_delta_net_test.cc:27-176, 299-340)."""
import math

import numpy as np

import oracle


def bf16(x: float) -> float:
    return float(oracle.round_bf16(np.array([x], np.float32))[0])


def make_example(length, kh, vh, kd, vd, kernel=3):
    """The reference test's closed-form inputs: 0.15 + 0.4 sin(0.37 i + 0.41 tensor), A_log
    shifted by -0.7, the norm weight by +1; activations (first four tensors) rounded to bf16;
    the upstream gradient is non-zero only at the last token."""
    channels = 2 * kh * kd + vh * vd
    sizes = [length * channels, length * vh * vd, length * vh, length * vh, channels * kernel,
             vh, vh, vd]
    values = []
    for tensor, n in enumerate(sizes):
        i = np.arange(n, dtype=np.float32)
        v = (np.float32(0.15) + np.float32(0.4) * np.sin(np.float32(0.37) * i + np.float32(0.41) * np.float32(tensor))).astype(np.float32)
        if tensor == 5:
            v = v - np.float32(0.7)
        if tensor == 7:
            v = v + np.float32(1.0)
        if tensor < 4:
            v = oracle.round_bf16(v)
        values.append(v.astype(np.float64))
    upstream = np.zeros(length * vh * vd, np.float32)
    i = np.arange((length - 1) * vh * vd, length * vh * vd, dtype=np.float32)
    upstream[(length - 1) * vh * vd:] = np.float32(0.4) * np.cos(np.float32(0.2) * i)
    return values, upstream


class DoubleModel:
    def __init__(self, length, kh, vh, kd, vd, kernel, eps, rnd):
        self.length, self.kh, self.vh, self.kd, self.vd = length, kh, vh, kd, vd
        self.kernel, self.eps, self.rnd = kernel, eps, rnd
        self.offsets, self.recording, self.index = [], False, 0

    def _round(self, x, enabled=None):
        if not (self.rnd if enabled is None else enabled):
            return x
        if self.recording:
            self.offsets.append(bf16(x) - x)
        x += self.offsets[self.index]
        self.index += 1
        return x

    def forward(self, v, record=False):
        """v: the eight tensors as flat lists (QKV, Z, A, B, conv, A_log, dt_bias, norm)."""
        self.recording, self.index = record, 0
        if record:
            self.offsets = []
        T, kh, vh, kd, vd, kernel = self.length, self.kh, self.vh, self.kd, self.vd, self.kernel
        channels = 2 * kh * kd + vh * vd
        conv = [0.0] * (T * channels)
        for t in range(T):
            for c in range(channels):
                s = 0.0
                for tap in range(kernel):
                    src = t + tap - kernel + 1
                    if src >= 0:
                        s += v[0][src * channels + c] * v[4][c * kernel + tap]
                s = self._round(s)
                conv[t * channels + c] = self._round(s / (1 + math.exp(-s)))
        states = [0.0] * (vh * kd * vd)
        core = [0.0] * (T * vh * vd)
        for head in range(vh):
            key_head = head // (vh // kh)
            for t in range(T):
                q = [conv[t * channels + key_head * kd + d] for d in range(kd)]
                k = [conv[t * channels + (kh + key_head) * kd + d] for d in range(kd)]
                qn = 1e-6 + sum(x * x for x in q)
                kn = 1e-6 + sum(x * x for x in k)
                q = [x / math.sqrt(qn * kd) for x in q]
                k = [x / math.sqrt(kn) for x in k]
                alpha = v[2][t * vh + head] + v[6][head]
                softplus = max(alpha, 0.0) + math.log1p(math.exp(-abs(alpha)))
                decay = math.exp(-math.exp(v[5][head]) * softplus)
                beta = self._round(1 / (1 + math.exp(-v[3][t * vh + head])))
                for ch in range(vd):
                    prediction = 0.0
                    for d in range(kd):
                        i = (head * kd + d) * vd + ch
                        states[i] *= decay
                        prediction += states[i] * k[d]
                    delta = (conv[t * channels + 2 * kh * kd + head * vd + ch] - prediction) * beta
                    out = 0.0
                    for d in range(kd):
                        i = (head * kd + d) * vd + ch
                        states[i] += k[d] * delta
                        out += states[i] * q[d]
                    core[(t * vh + head) * vd + ch] = self._round(out)
        result = [0.0] * len(core)
        for row in range(T * vh):
            ss = sum(core[row * vd + d] ** 2 for d in range(vd))
            inverse = 1 / math.sqrt(ss / vd + self.eps)
            for d in range(vd):
                i = row * vd + d
                normalized = self._round(core[i] * inverse)
                affine = self._round(normalized * v[7][d])
                result[i] = self._round(affine * v[1][i] / (1 + math.exp(-v[1][i])), True)
        return result

    def gradients(self, values, upstream, step=1e-5):
        values = [list(map(float, x)) for x in values]
        self.forward(values, record=True)

        def loss():
            y = self.forward(values)
            return sum(p * q for p, q in zip(y, upstream))

        grads = []
        for tensor in range(len(values)):
            g = []
            for i in range(len(values[tensor])):
                original = values[tensor][i]
                values[tensor][i] = original + step
                plus = loss()
                values[tensor][i] = original - step
                minus = loss()
                values[tensor][i] = original
                g.append((plus - minus) / (2 * step))
            grads.append(np.array(g))
        return grads
