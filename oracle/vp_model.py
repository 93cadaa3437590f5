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


class NumpyFastCompute(NumpyCompute):
    """Adds the stages of the 3-collective protocol (candidate lists, one all-gather, redundant finish on every rank).

    Same regions and same meaning of every reduced number as the CUDA kernels; the per-shard arithmetic is the plain
    numpy statement (whole shard in sub-block 0, exact octave histogram)."""
    BINS = 32

    def _e(self):
        gmax = self.s.f_stat1.numpy().reshape(self.s.B, -1).max(axis=1)
        return np.exp2(self._x() - gmax[:, None]).astype(np.float32)

    def _stat2(self):
        s = self.s
        return s.f_stat2.numpy().reshape(s.B, -1, 2 + 2 * self.BINS)

    def _denom_bound(self):
        st = self._stat2()
        denom = st[:, :, 0].sum(axis=1, dtype=np.float32)
        bound = np.zeros(self.s.B, dtype=np.float32)
        for b in range(self.s.B):
            cm = cc = np.float32(0)
            for k in range(self.BINS):
                cm = np.float32(cm + st[b, :, 2 + 2 * k].sum(dtype=np.float32))
                cc = np.float32(cc + st[b, :, 3 + 2 * k].sum(dtype=np.float32))
                if cc > self.fk + 1 or cm > np.float32(self.top_p * denom[b]) * np.float32(1.001):
                    bound[b] = np.float32(2.0 ** -(k + 1))
                    break
        return denom, bound

    def stage(self, name, rnd=0):
        s = self.s
        B = s.B
        if name == "f_max":
            s.f_stat1.numpy().reshape(B, -1)[:] = self._x().max(axis=1)[:, None]
            s.f_all_valid.numpy()[0] = 1
        elif name == "f_sum":
            e = self._e()
            st = self._stat2()
            st[:] = 0
            st[:, 0, 0] = e.sum(axis=1, dtype=np.float32)
            with np.errstate(divide="ignore"):
                k = np.floor(-np.log2(e.astype(np.float64)))          # e in (2^-(k+1), 2^-k]
            k = np.where(e >= 1, 0, np.where(np.exp2(-k) == e, k - 1, k))
            for b in range(B):
                for kk in range(self.BINS):
                    m = k[b] == kk
                    st[b, 0, 2 + 2 * kk] = e[b][m].sum(dtype=np.float32)
                    st[b, 0, 3 + 2 * kk] = np.float32(m.sum())
        elif name == "f_extract":
            e = self._e()
            _, bound = self._denom_bound()
            self._lists = [np.nonzero(e[b] >= bound[b])[0] if bound[b] > 0 else None for b in range(B)]
            self._evals = e
        elif name == "f_compact":
            lmax = s.f_send.numel() // (2 * B)
            send = s.f_send.numpy().view(np.uint32).reshape(B, lmax, 2)
            cnt = s.f_send_cnt.numpy().view(np.uint32).reshape(B, -1)     # one count per segment; the model fills segment 0 only
            cnt[:] = 0
            seg = lmax // cnt.shape[1]
            for b in range(B):
                idx = self._lists[b]
                if idx is None or len(idx) > seg:
                    cnt[b, 0] = 0xffffffff
                    continue
                cnt[b, 0] = len(idx)
                send[b, :len(idx), 0] = self._evals[b][idx].view(np.uint32)
                send[b, :len(idx), 1] = (idx + s.col0).astype(np.uint32)
        elif name == "f_finish":
            lmax = s.f_send.numel() // (2 * B)
            gath = s.f_gath.numpy().view(np.uint32).reshape(s.world, B, lmax, 2)
            gcnt = s.f_gath_cnt.numpy().view(np.uint32).reshape(s.world, B, -1)
            seg = lmax // gcnt.shape[2]
            gcnt = gcnt[:, :, 0]
            denom, bound = self._denom_bound()
            ids, valid = s.f_ids.numpy(), s.f_valid.numpy()
            for b in range(B):
                ok = bool(bound[b] > 0) and bool((gcnt[:, b] <= seg).all())
                parts = [gath[r, b, :min(int(gcnt[r, b]), seg)] for r in range(s.world)]
                ent = np.concatenate(parts, axis=0)
                p = (ent[:, 0].copy().view(np.float32) / denom[b]).astype(np.float32)
                pb = p.view(np.uint32).astype(np.uint64)
                left = np.uint64(np.float32(bound[b] / denom[b]).view(np.uint32)) + np.uint64(1)
                right = np.uint64(0x3f800001)

                def passes(piv):
                    m = pb >= piv
                    return (np.float32(m.sum()) < self.fk) and (p[m].sum(dtype=np.float32) < self.fp)
                if passes(left):
                    ok = False
                for _ in range(8):
                    w = right - left
                    if w <= 1:
                        break
                    nl, nr, found = left, right, False
                    for j in range(P):
                        piv = left + ((w * np.uint64(j + 1)) >> np.uint64(4))
                        if not passes(piv):
                            nl = piv
                        elif not found:
                            nr, found = piv, True
                    left, right = nl, nr
                thr = np.uint32(left).view(np.float32)
                gt, eq = p > thr, p == thr
                sgtk, sgtp, seqk = np.float32(gt.sum()), p[gt].sum(dtype=np.float32), np.float32(eq.sum())
                comp = np.float32(1)
                if seqk > 0:
                    if self.use_p:
                        with np.errstate(all="ignore"):
                            comp = min(_sf(np.float32((self.top_p - sgtp) / (thr * seqk))), comp)
                    comp = max(min(_sf(np.float32((self.fk - sgtk) / seqk)), comp), np.float32(0))
                wgt = np.where(p < thr, np.float32(0), np.where(eq, p * comp, p)).astype(np.float32)
                tmp = self.states.copy()
                u = np.float32(co.uniform(co.draw4(tmp, b)[0]))
                cum = np.cumsum(wgt, dtype=np.float32)
                target = np.float32(cum[-1] * u) if len(cum) else np.float32(0)
                hit = np.nonzero((wgt > 0) & (target <= cum))[0]
                kept = np.nonzero(wgt > 0)[0]
                if len(kept) == 0:
                    ids[b], valid[b] = 1, 0
                    s.f_all_valid.numpy()[0] = 0
                    continue
                pos = hit[0] if len(hit) else kept[-1]
                ids[b] = int(ent[pos, 1]) + 1
                valid[b] = 1 if ok else 0
                if not ok:
                    s.f_all_valid.numpy()[0] = 0
                self._thr = getattr(self, "_thr", dict())
                self._thr[b] = thr
        elif name == "f_advance":
            if s.f_all_valid.numpy()[0] == 0:
                return
            for b in range(B):
                co.draw4(self.states, b)
        elif name == "penalty" and rnd == 1:
            if s.f_all_valid.numpy()[0] == 0:
                return
            keep = s.ids.numpy().copy()
            s.ids.numpy()[:] = s.f_ids.numpy()
            super().stage("penalty")
            s.ids.numpy()[:] = keep
        else:
            super().stage(name, rnd)
