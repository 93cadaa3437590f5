"""numpy model of one shard's arithmetic in vocab-parallel sampling.  TEST INFRASTRUCTURE ONLY.

Implements the ``compute`` interface of ``rapid_sampling_b200.vocab_parallel.VocabParallelSampler`` (``bind`` +
``stage``) on CPU tensors, so that the driver's sequence of stages and collectives can run among gloo ranks
without a GPU.  The semantics are those of the reference kernels on the union of the shards (sampling.cu:517-752):
kept set {p >= v}, fractional weight ``comp`` for the ties with v (sampling.cu:690-696), in-place penalty update
(sampling.cu:427-437).  The search is the driver's own 16-ary search over fp32 bit patterns.
"""
import numpy as np

from . import c_oracle as co

FLT_MAX = np.float32(3.4028234663852886e38)
P = 15


def _sf(x):
    x = np.where(np.isnan(x), np.float32(0), x)
    return np.clip(x, -FLT_MAX, FLT_MAX).astype(np.float32)


class NumpyCompute:
    def bind(self, s, logits, states, penalties, temperature, top_k, top_p, presence, repetition, decay):
        self.s = s
        lg = logits.numpy()
        self.lg = lg[:, -1, :] if lg.ndim == 3 else lg
        self.states = states.numpy()
        self.pen = penalties.numpy() if penalties is not None else None
        V = s.V_global
        if top_k <= 0 or top_k > V:
            top_k = V
        if top_p < 0 or top_p > 1:
            top_p = 1.0
        if top_p == 0:
            top_k, top_p = 1, 1.0
        self.use_p = top_p < 1.0
        self.fk = np.float32(top_k)
        self.fp = np.float32(top_p) if self.use_p else np.float32(np.inf)
        self.top_p = np.float32(top_p)
        self.scale = np.float32(1.4426950408889634074 / temperature)
        self.presence, self.repetition, self.decay = np.float32(presence), np.float32(repetition), np.float32(decay)

    def _x(self):
        l = _sf(self.lg.astype(np.float32))
        if self.pen is not None:
            l = l - self.pen
        return _sf(l * self.scale)

    def _p(self):
        s = self.s
        e = np.exp2(self._x() - s.gmax.numpy()[:, None]).astype(np.float32)
        return (e / s.gsum.numpy()[:, None]).astype(np.float32)

    def _bracket(self, rounds_done):
        s = self.s
        B = s.B
        left = np.zeros(B, dtype=np.uint64)
        right = np.full(B, 0x3f800001, dtype=np.uint64)
        for r in range(rounds_done):
            t = s.tallies[r].numpy().reshape(B, P, 2)
            for b in range(B):
                if right[b] - left[b] <= 1:
                    continue
                w = right[b] - left[b]
                piv = [left[b] + ((w * (j + 1)) >> np.uint64(4)) for j in range(P)]
                nl, nr, found = left[b], right[b], False
                for j in range(P):
                    ok = (t[b, j, 0] < self.fk) and (t[b, j, 1] < self.fp)
                    if not ok:
                        nl = piv[j]
                    elif not found:
                        nr, found = piv[j], True
                left[b], right[b] = nl, nr
        return left.astype(np.uint32), right.astype(np.uint32)

    def _comp(self, thr):
        g = self.s.gtally.numpy().reshape(self.s.B, 4)
        comp = np.ones(self.s.B, dtype=np.float32)
        for b in range(self.s.B):
            sgtk, sgtp, seqk = g[b, 0], g[b, 1], g[b, 2]
            if seqk > 0:
                c = np.float32(1.0)
                if self.use_p:
                    with np.errstate(all="ignore"):
                        c = min(_sf(np.float32((self.top_p - sgtp) / (thr[b] * seqk))), c)
                c = min(_sf(np.float32((self.fk - sgtk) / seqk)), c)
                comp[b] = max(c, np.float32(0))
        return comp

    def _weights(self, p, thr, comp):
        return np.where(p < thr[:, None], np.float32(0), np.where(p == thr[:, None], p * comp[:, None], p)).astype(np.float32)

    def stage(self, name, rnd=0):
        s = self.s
        B = s.B
        if name == "max":
            s.gmax.numpy()[:] = self._x().max(axis=1)
        elif name == "sum":
            s.gsum.numpy()[:] = np.exp2(self._x() - s.gmax.numpy()[:, None]).astype(np.float32).sum(axis=1, dtype=np.float32)
        elif name == "round":
            left, right = self._bracket(rnd)
            pb = self._p().view(np.uint32)
            p = pb.view(np.float32)
            out = s.tallies[rnd].numpy().reshape(B, P, 2)
            out[:] = 0
            for b in range(B):
                w = np.uint64(right[b]) - np.uint64(left[b])
                if w <= 1:
                    continue
                for j in range(P):
                    piv = np.uint32(np.uint64(left[b]) + ((w * np.uint64(j + 1)) >> np.uint64(4)))
                    m = pb[b] >= piv
                    out[b, j, 0] = np.float32(m.sum())
                    out[b, j, 1] = p[b][m].sum(dtype=np.float32)
        elif name == "tally":
            left, _ = self._bracket(len(s.tallies))
            pb = self._p().view(np.uint32)
            p = pb.view(np.float32)
            out = s.gtally.numpy().reshape(B, 4)
            for b in range(B):
                gt = pb[b] > left[b]
                out[b] = (gt.sum(), p[b][gt].sum(dtype=np.float32), (pb[b] == left[b]).sum(), 0)
        elif name == "weight":
            left, _ = self._bracket(len(s.tallies))
            thr = left.view(np.float32)
            w = self._weights(self._p(), thr, self._comp(thr))
            out = s.weights.numpy().reshape(B, s.world)
            out[:] = 0
            out[:, s.rank] = w.sum(axis=1, dtype=np.float32)
        elif name == "pick":
            left, _ = self._bracket(len(s.tallies))
            thr = left.view(np.float32)
            w = self._weights(self._p(), thr, self._comp(thr))
            W = s.weights.numpy().reshape(B, s.world)
            ids = s.ids.numpy()
            for b in range(B):
                u = np.float32(co.uniform(co.draw4(self.states, b)[0]))
                target = np.float32(W[b].sum(dtype=np.float32) * u)
                run, owner, before, last, before_last = np.float32(0), -1, np.float32(0), 0, np.float32(0)
                for k in range(s.world):
                    if W[b, k] > 0:
                        last, before_last = k, run
                    nxt = np.float32(run + W[b, k])
                    if owner < 0 and W[b, k] > 0 and target <= nxt:
                        owner, before = k, run
                    run = nxt
                if owner < 0:
                    owner, before = last, before_last
                if owner != s.rank:
                    ids[b] = 0
                    continue
                cum = before + np.cumsum(w[b], dtype=np.float32)
                hit = np.nonzero((w[b] > 0) & (target <= cum))[0]
                idx = hit[0] if len(hit) else np.nonzero(w[b] > 0)[0][-1]
                ids[b] = s.col0 + idx + 1
        elif name == "penalty":
            ids = s.ids.numpy() - 1
            old = self.pen.copy()
            new = (old * self.decay).astype(np.float32)
            for b in range(B):
                c = ids[b] - s.col0
                if 0 <= c < s.V_local:
                    new[b, c] = np.float32(old[b, c] * self.decay + (self.presence if old[b, c] == 0 else self.repetition))
            self.pen[:] = new
        else:
            raise ValueError(name)
