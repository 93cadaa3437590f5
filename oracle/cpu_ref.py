"""float64 torch-CPU statement of the sampler's semantics.  TEST INFRASTRUCTURE ONLY.

Closed form of what the reference kernels compute (sampling.cu:517-752; penalties :220, :427-437;
argument remaps :1005-1010): softmax over the penalised, temperature-scaled logits; sort; the kept
set is every token whose probability is >= v, where v is the probability of the n-th largest token
and n = min(top_k, first rank whose cumulative mass reaches top_p).  Tokens strictly above v keep
their full weight; tokens EQUAL to v are scaled by ``comp`` so that the kept mass equals top_p /
the kept count equals top_k exactly (sampling.cu:365-371, :690-696).  ``top_p >= 1`` means "no
top-p constraint" (the kernels never measure the mass of the full set, sampling.cu:596).

Unlike ``sampler_oracle.c`` this makes no attempt to follow the kernels' fp32 operation order; it is
the independent semantic check (kept set, weights, chi-square expectation) and the float64 CPU path
timed as a baseline.
"""
import math

import torch

FLT_MAX = 3.4028234663852886e38
LOG2E = 1.4426950408889634074


def _sf(x):
    x = torch.nan_to_num(x, nan=0.0, posinf=FLT_MAX, neginf=-FLT_MAX)
    return x


def normalise(V, temperature, top_k, top_p):
    """Argument remaps of sampling.cu:1005-1011 (values as the kernels see them, fp32-rounded)."""
    if not (V > 0 and V <= 1048576 and V % 4 == 0):
        raise ValueError("Vocabulary size must be multiple of 4, and no larger than 1048576")
    if not (temperature >= 0.001 and temperature <= 1000):
        raise ValueError("Temperature outside range")
    if top_k <= 0 or top_k > V:
        top_k = V
    if top_p < 0 or top_p > 1:
        top_p = 1.0
    if top_p == 0:
        top_k, top_p = 1, 1.0
    scale = float(torch.tensor(LOG2E / temperature, dtype=torch.float64).float())
    top_p32 = float(torch.tensor(top_p, dtype=torch.float64).float())
    return scale, int(top_k), top_p32


def distribution(logits, temperature, top_k, top_p, penalties=None):
    """logits (B,V) fp32 CPU tensor -> dict of float64 tensors: probs, weights (un-normalised sampling
    weights, zero outside the kept set), kept (bool), v (threshold prob per row), comp, cum_sorted, order."""
    assert logits.dim() == 2
    B, V = logits.shape
    scale, k, p = normalise(V, temperature, top_k, top_p)
    x = _sf(logits.float()).double()
    if penalties is not None:
        x = x - penalties.double()
    x = _sf(x * scale)                              # log2 units
    probs = torch.softmax(x * math.log(2.0), dim=-1)
    sp, order = torch.sort(probs, dim=-1, descending=True, stable=True)
    cum = torch.cumsum(sp, dim=-1)
    if p >= 1.0:
        n_p = torch.full((B,), V, dtype=torch.long)
    else:
        n_p = (cum < p).sum(dim=-1) + 1             # first rank whose cumulative mass >= p
        n_p = torch.clamp(n_p, max=V)
    n = torch.clamp(n_p, max=k)
    v = sp.gather(1, (n - 1).unsqueeze(1))          # (B,1)
    gt = probs > v
    eq = probs == v
    m = eq.sum(dim=-1).double()
    mass_gt = (probs * gt).sum(dim=-1)
    cnt_gt = gt.sum(dim=-1).double()
    c1 = (p - mass_gt) / (v.squeeze(1) * m) if p < 1.0 else torch.full((B,), float("inf"), dtype=torch.float64)
    c2 = (k - cnt_gt) / m
    comp = torch.clamp(torch.minimum(torch.minimum(c1, c2), torch.ones(B, dtype=torch.float64)), min=0.0)
    weights = torch.where(gt, probs, torch.where(eq, probs * comp.unsqueeze(1), torch.zeros_like(probs)))
    return {"probs": probs, "weights": weights, "kept": gt | eq, "v": v.squeeze(1), "comp": comp,
            "cum_sorted": cum, "sorted": sp, "order": order, "n": n, "top_k": k, "top_p": p}


def sample(logits, temperature, top_k, top_p, penalties=None, presence=0.0, repetition=0.0, decay=0.0,
           generator=None):
    """One sampling call on CPU in float64 (inverse-CDF over the weights); updates penalties in place.
    logits: (V,), (B,V) or (B,T,V) -- only position T-1 is read (sampling.cu:202). Returns int64 ids (B,)."""
    if logits.dim() == 1:
        logits = logits.unsqueeze(0)
    if logits.dim() == 3:
        logits = logits[:, -1, :]
    d = distribution(logits, temperature, top_k, top_p, penalties)
    ids = torch.multinomial(d["weights"], 1, generator=generator).squeeze(1)
    if penalties is not None:
        hit = torch.zeros_like(penalties)
        old = penalties.gather(1, ids.unsqueeze(1))
        hit.scatter_(1, ids.unsqueeze(1), torch.where(old == 0, torch.tensor(presence), torch.tensor(repetition)).float())
        penalties.mul_(decay).add_(hit)
    return ids
