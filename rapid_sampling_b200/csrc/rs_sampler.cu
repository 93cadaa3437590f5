// Token sampler for B200 (sm_100a): penalties/temperature -> softmax -> top-k/top-p cutoff ->
// one sampled id per row, bit-compatible with the reference kernels (sampling.cu:172-438,
// :517-752, :757-964) but organised differently:
//
//   * a row is handled by a thread-block CLUSTER of C CTAs (C = 1..16).  The reference's 1024
//     threads become 1024 "virtual lanes"; CTA c plays lanes [c*1024/C, (c+1)*1024/C).  Lane t
//     still owns float4 groups t, t+1024, ... so every fp32 sum keeps the reference's order.
//   * on-chip variant (small batches): the row is read from HBM ONCE, by 1-D bulk async copies (one per
//     stripe) into the cluster's shared memory, and all later passes run on chip.  Streaming variant
//     (batches beyond what is resident at once): the row is read twice (HBM, then L2) and only a short
//     candidate list stays on chip.  The reference re-reads a global scratch copy ~18 times from one SM.
//   * candidate list: a bound derived from the threads' own maxima selects the ~200 largest elements of
//     the row; the cutoff search replays the reference's pivots on that list and proves for each pivot
//     that the decision equals the one taken on the whole row.  Rows whose list cannot settle the cutoff
//     fall back to the search over the whole row, which drops, in place and order-preserving, every element
//     below the current lower bound as the bracket rises.
//   * warp partials cross CTAs through small distributed-shared-memory mailboxes (remote vector stores that
//     count their bytes on an mbarrier of the destination, no cluster barrier); every CTA combines the 32
//     partials itself in the reference's order, so all CTAs take identical decisions without a broadcast.
//   * rows too large for the cluster's shared memory use the same code on a global scratch row.
//
// No tensor cores: nothing here is a contraction.  The bound is HBM bandwidth (4 bytes per
// logit, 12 with penalties) for large batches and launch + barrier latency for tiny ones.
#include "rs_common.cuh"
#include "rs_rowcta.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "../../include/rapid_sampling_b200.h"

#include <atomic>
#include <cstdio>
#include <cstring>
#include <initializer_list>
#include <mutex>

namespace rs {

// CTAs of one variant that the register file of an SM holds (64K registers): the streaming variant is compiled
// for 64 registers per thread, the on-chip variants for up to 128.  The launch planner counts resident rows with it.
__host__ __device__ constexpr int ctas_per_sm_by_registers(int C, bool smem_variant) {
    return smem_variant ? (C >= 4 ? C / 2 : 1) : (C == 8 ? 8 : 1);
}

// MORE_REGS (streaming variant only): compiled for 6 CTAs per SM (80 registers) instead of 8 (64): no spills and twice
// the loads in flight per thread, for batches whose CTAs fit the GPU at 6 per SM anyway.
template <int C, bool SMEM, bool LOWP, bool ROWP, bool MORE_REGS = false>
__global__ void __launch_bounds__(kLanes / C, MORE_REGS ? 6 : ctas_per_sm_by_registers(C, SMEM)) sampler_kernel(const Params p) {
    constexpr int L = kLanes / C;
    constexpr int WPC = L / 32;  // warps per CTA
    constexpr unsigned FULL = 0xffffffffu;
    extern __shared__ __align__(128) unsigned char smem[];
    const int t = threadIdx.x, lane = t & 31, wl = t >> 5;
    const uint32_t crank = (C == 1) ? 0u : cluster_ctarank();
    const int b = blockIdx.x / C;
    const int tg = (int)crank * L + t;  // virtual lane
    const int wg = tg >> 5;             // virtual warp
    const int V = p.V, V4 = V >> 2;
    const int Kt = (tg < V4) ? ((V4 - tg + kLanes - 1) >> 10) : 0;
    // Programmatic dependent launch: the next kernel in the stream may be set up while this one runs, and this one may
    // have been set up while its predecessor ran -- nothing in global memory is touched before the predecessor is
    // complete and visible.
    grid_dependents_may_launch();
    grid_dependency_wait();
    // per-call parameters, or (ROWP) this row's own
    int a_kind = p.kind, a_top_k = p.top_k, a_sel_rank = p.sel_rank;
    float a_scale = p.scale, a_top_p = p.top_p;
    if (ROWP) {
        const RowArgs ra = p.rows[b];
        a_kind = ra.kind; a_top_k = ra.top_k; a_sel_rank = ra.sel_rank; a_scale = ra.scale; a_top_p = ra.top_p;
    }
    const bool rep = (a_kind == kRepetition);
    const bool use_cnt = (a_kind != kTopP);
    const int dtype = LOWP ? p.dtype : RS_DTYPE_F32;   // fp32 rows keep a kernel of their own: no type tests in its loops
    const char* lrow_b = reinterpret_cast<const char*>(p.logits) + (long long)b * p.row_stride * (dtype == RS_DTYPE_F32 ? 4 : 2);
    const float* lrow = reinterpret_cast<const float*>(lrow_b);   // valid as such for fp32 logits only
    // four consecutive logits (group g of the row) / one logit, converted exactly to fp32
    auto ldrow4 = [&](int g) -> float4 {
        if (!LOWP) return __ldg(reinterpret_cast<const float4*>(lrow_b) + g);
        const uint2 r = __ldg(reinterpret_cast<const uint2*>(lrow_b) + g);
        if (dtype == RS_DTYPE_F16) {
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
            const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
            return make_float4(a.x, a.y, c.x, c.y);
        }
        return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u), __uint_as_float(r.y << 16),
                           __uint_as_float(r.y & 0xffff0000u));
    };
    auto ldrow1 = [&](int i) -> float {
        if (!LOWP) return reinterpret_cast<const float*>(lrow_b)[i];
        const unsigned short h = reinterpret_cast<const unsigned short*>(lrow_b)[i];
        if (dtype == RS_DTYPE_F16) return __half2float(__ushort_as_half(h));
        return __uint_as_float((uint32_t)h << 16);
    };
    constexpr bool bulk_load = SMEM && !LOWP;   // 16-bit logits are staged through registers
    float* prow = rep ? p.penalties + (long long)b * V : nullptr;

    uint64_t* mbar = reinterpret_cast<uint64_t*>(smem + kMiscOff);
    uint64_t* xbar = reinterpret_cast<uint64_t*>(smem + kMiscOff + 16);   // two mailbox barriers
    int* s_idxt = reinterpret_cast<int*>(smem + kMiscOff + 8);
    int* s_token = reinterpret_cast<int*>(smem + kMiscOff + 12);
    float* s_wtot = reinterpret_cast<float*>(smem + kMiscOff + 64);
    volatile uint32_t* s_res = reinterpret_cast<volatile uint32_t*>(smem + kMiscOff + 192);   // ten combined words of an exchange
    volatile int* s_fail = reinterpret_cast<volatile int*>(smem + kMiscOff + 32);             // set when a bounded wait of this CTA gave up
    uint64_t* qbar = reinterpret_cast<uint64_t*>(smem + kMiscOff + 40);                       // counts the bytes of the unordered candidate list
    volatile uint32_t* s_quick = reinterpret_cast<volatile uint32_t*>(smem + kMiscOff + 48);  // outcome of the one-warp search: left, right, rounds, verdict
    uint2* qlist = reinterpret_cast<uint2*>(smem + kQuickOff);
    // A wait that ran out: the status word (and its host mirror) say so, and this CTA stops producing results --
    // its row reports id -1 and leaves the RNG state and the penalties as they were.
    auto wait_failed = [&]() {
        atomicExch(p.status, RS_ERR_TIMEOUT);
        if (p.status_mirror) *reinterpret_cast<volatile int*>(p.status_mirror) = RS_ERR_TIMEOUT;
        *s_fail = 1;
    };
    Row<C, SMEM> row;
    row.slab = SMEM ? reinterpret_cast<float4*>(smem + kSlabOff + p.cand_slots * L * 16)
                    : reinterpret_cast<float4*>(p.scratch + (long long)b * V);
    row.t = t;
    row.tg = tg;
    // candidate buffer: cand_slots float4 slots per lane, [slot][lane] like the slab
    float* cand = reinterpret_cast<float*>(smem + kSlabOff);
    const int cap = p.cand_slots * 4;
    auto cand_at = [&](int i) -> float& { return cand[((i >> 2) * L + t) * 4 + (i & 3)]; };

    // x = sanitised scaled logit of slot s: kept in the shared-memory stripes, or (streaming variant) read
    // again from global memory -- the same functions on the same inputs, hence the same bits
    auto xload = [&](int s) -> float4 {
        if (SMEM) return row.ld(s);
        float4 v = ldrow4(s * kLanes + tg);
        if (rep) {
            const float4 q4 = __ldcg(reinterpret_cast<const float4*>(prow) + s * kLanes + tg);
            v = scaled4_rep(v, q4, a_scale);
        } else {
            v = scaled4(v, a_scale);
        }
        return v;
    };
    // ---- exchange of warp values across the cluster ----------------------------------------------------
    // Every warp contributes kXWords words; word k of (virtual) warp w lands at box[w * kXStride + k] in EVERY
    // CTA's mailbox.  Lane l supplies word l >> 3 (a), word 4 + (l >> 3) (b) and, for l < 16, word 8 + (l >> 3)
    // (c); the words are first collected in the lanes that send (lane r serves CTA r), so that a warp's record
    // travels as three vector stores per destination instead of ten scalar ones.  The stores count their bytes
    // on an mbarrier of the destination CTA, so a CTA only waits for its own mailbox to fill (bounded poll) --
    // no cluster-wide barrier.  Two mailboxes alternate: a CTA can post exchange n+2 only after it has received
    // everybody's n+1, which each CTA sends after it has finished reading n.
    int phase = 0;
    uint32_t xpar = 0;
    auto exchange = [&](auto packets, uint32_t a, uint32_t bq, uint32_t c2, const bool wait_here = true) -> const uint32_t* {
        constexpr int NP = decltype(packets)::value;   // 1: words 0-3 (a); 2: + words 4-7 (b); 3: + words 8-9 (c)
        uint32_t* box = reinterpret_cast<uint32_t*>(smem + kMboxOff + phase * kMboxBuf);
        uint32_t wa[4], wb[4] = {0u, 0u, 0u, 0u}, wc[2] = {0u, 0u};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            wa[k] = __shfl_sync(FULL, a, k * 8);
            if (NP >= 2) wb[k] = __shfl_sync(FULL, bq, k * 8);
        }
        if (NP >= 3) {
            wc[0] = __shfl_sync(FULL, c2, 0);
            wc[1] = __shfl_sync(FULL, c2, 8);
        }
        if (C == 1) {
            if (lane == 0) {
                uint4* rec = reinterpret_cast<uint4*>(box + wg * kXStride);
                rec[0] = make_uint4(wa[0], wa[1], wa[2], wa[3]);
                if (NP >= 2) rec[1] = make_uint4(wb[0], wb[1], wb[2], wb[3]);
                if (NP >= 3) *reinterpret_cast<uint2*>(rec + 2) = make_uint2(wc[0], wc[1]);
            }
            __syncthreads();
        } else {
            const uint32_t bar = smem_addr(xbar + phase);
            if (t == 0) mbar_expect_tx(bar, (uint32_t)((NP == 1 ? 4 : NP == 2 ? 8 : kXWords) * 32 * 4));
            if (lane < C) {
                const uint32_t dst = map_to_cta(smem_addr(box + wg * kXStride), (uint32_t)lane);
                const uint32_t rbar = map_to_cta(bar, (uint32_t)lane);
                st_async_v4(dst, wa[0], wa[1], wa[2], wa[3], rbar);
                if (NP >= 2) st_async_v4(dst + 16, wb[0], wb[1], wb[2], wb[3], rbar);
                if (NP >= 3) st_async_v2(dst + 32, wc[0], wc[1], rbar);
            }
            if (wait_here && !mbar_wait_bounded(bar, (xpar >> phase) & 1u, p.wait_polls)) wait_failed();
        }
        xpar ^= (1u << phase);
        phase ^= 1;
        return box;
    };
    // word k of virtual warp w in a mailbox
    auto bx = [&](const uint32_t* box, int k, int w) -> uint32_t { return box[w * kXStride + k]; };
    const int xk = lane >> 3;   // which of four values this lane forwards
    auto pick4 = [&](uint32_t v0, uint32_t v1, uint32_t v2, uint32_t v3) -> uint32_t {
        return xk == 0 ? v0 : xk == 1 ? v1 : xk == 2 ? v2 : v3;
    };
    // phase timestamps (ns) for the trace: test instrumentation only
    uint32_t ts[10];
    const bool want_ts = (p.dbg_trace != nullptr);
    unsigned long long t_begin = 0;
    auto stamp = [&](int i) {
        if (want_ts) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (i == 0) t_begin = now;
            ts[i] = (uint32_t)(now - t_begin);
        }
    };
#pragma unroll
    for (int i = 0; i < 10; i++) ts[i] = 0;
    stamp(0);

    // Row totals of four ordered masses and four counts (packed per lane as c01 = n0 | n1 << 16,
    // c23 = n2 | n3 << 16; a lane holds at most 1024 elements), plus min / max of two bit patterns.
    // Order of the masses: xor tree over the 32 lanes of a warp (offsets 16, 8, 4, 2, 1), then the 32 warp
    // values added in warp order, as thread 0 of the reference does (sampling.cu:34-42).  The four trees
    // share shuffles: at offsets 16 and 8 a lane keeps half of the sums and hands the other half to its
    // partner -- the same additions as four separate butterflies -- so that lane l ends with sum l >> 3.
    // Every warp of every CTA then combines the 32 mailbox columns itself: lanes 0..7 run the eight
    // 32-step chains (counts travel as exact floats), so no second synchronisation is needed.
    auto totals = [&](const float (&m)[4], uint32_t c01, uint32_t c23, uint32_t mn, uint32_t mxv, uint32_t (&cnt)[4],
                      float (&mass)[4], uint32_t& vmin, uint32_t& vmax) {
        float x;
        {
            const bool up16 = (lane & 16) != 0, up8 = (lane & 8) != 0;
            const float a0 = (up16 ? m[2] : m[0]) + __shfl_xor_sync(FULL, up16 ? m[0] : m[2], 16);
            const float a1 = (up16 ? m[3] : m[1]) + __shfl_xor_sync(FULL, up16 ? m[1] : m[3], 16);
            x = (up8 ? a1 : a0) + __shfl_xor_sync(FULL, up8 ? a0 : a1, 8);
            x = x + __shfl_xor_sync(FULL, x, 4);
            x = x + __shfl_xor_sync(FULL, x, 2);
            x = x + __shfl_xor_sync(FULL, x, 1);
        }
        c01 = __reduce_add_sync(FULL, c01);
        c23 = __reduce_add_sync(FULL, c23);
        mn = __reduce_min_sync(FULL, mn);
        mxv = __reduce_max_sync(FULL, mxv);
        const float cf = __uint2float_rn(pick4(c01 & 0xffffu, c01 >> 16, c23 & 0xffffu, c23 >> 16));
        // Only the first warp of a CTA waits for the mailbox and combines it; the others pick the ten results up
        // from shared memory after a CTA barrier instead of repeating the 32-step chains.
        const uint32_t* box = exchange(Packets<3>(), __float_as_uint(x), __float_as_uint(cf), xk == 0 ? mn : mxv, wl == 0);
        if (wl == 0) {
            const uint32_t bmin = __reduce_min_sync(FULL, bx(box, 8, lane));
            const uint32_t bmax = __reduce_max_sync(FULL, bx(box, 9, lane));
            float sacc = 0.f;
            if (lane < 8) {
                sacc = __uint_as_float(bx(box, lane, 0));
#pragma unroll
                for (int w = 1; w < kWarps; w++) sacc += __uint_as_float(bx(box, lane, w));
                s_res[lane] = __float_as_uint(sacc);
            }
            if (lane == 8) s_res[8] = bmin;
            if (lane == 9) s_res[9] = bmax;
        }
        __syncthreads();
        {
            const uint32_t* rp = const_cast<const uint32_t*>(s_res);   // ordered by the barrier above
            const uint4 r0 = *reinterpret_cast<const uint4*>(rp), r1 = *reinterpret_cast<const uint4*>(rp + 4);
            const uint2 r2 = *reinterpret_cast<const uint2*>(rp + 8);
            mass[0] = __uint_as_float(r0.x); mass[1] = __uint_as_float(r0.y); mass[2] = __uint_as_float(r0.z);
            mass[3] = __uint_as_float(r0.w);
            cnt[0] = __float2uint_rn(__uint_as_float(r1.x)); cnt[1] = __float2uint_rn(__uint_as_float(r1.y));
            cnt[2] = __float2uint_rn(__uint_as_float(r1.z)); cnt[3] = __float2uint_rn(__uint_as_float(r1.w));
            vmin = r2.x;
            vmax = r2.y;
        }
    };

    // ---- load: bulk async copies of this CTA's stripes; RNG state read meanwhile -------------
    if (SMEM) {
        if (t == 0) {
            mbar_init(smem_addr(mbar), 1);
            mbar_init(smem_addr(xbar), 1);
            mbar_init(smem_addr(xbar + 1), 1);
            mbar_init(smem_addr(qbar), 1);
            fence_mbar_init();
            *s_idxt = 0;
            *s_token = 0;
            *s_fail = 0;
        }
        __syncthreads();
        if (bulk_load) {
            // One copy per stripe, issued by as many threads as there are stripes: a warp issues its lanes' copies one
            // after the other (64 copies from one warp took 1.9 us), so they are spread over all warps of the CTA.
            const int kfull = V4 >> 10, rem = V4 & 1023;
            const int vl = min(max(rem - (int)crank * L, 0), L);
            const uint32_t bar = smem_addr(mbar);
            if (t == 0) mbar_expect_tx(bar, (uint32_t)(kfull * L + vl) * 16u);
            const float4* src = reinterpret_cast<const float4*>(lrow) + crank * L;
            const uint32_t dst = smem_addr(row.slab);
            for (int k = lane * WPC + wl; k < kfull; k += L)      // consecutive stripes go to different warps
                bulk_g2s(dst + k * L * 16, src + k * kLanes, L * 16, bar);
            if (t == L - 1 && vl > 0) bulk_g2s(dst + kfull * L * 16, src + kfull * kLanes, vl * 16, bar);
        }
    } else {
        if (t == 0) {
            mbar_init(smem_addr(xbar), 1);
            mbar_init(smem_addr(xbar + 1), 1);
            mbar_init(smem_addr(qbar), 1);
            fence_mbar_init();
            *s_idxt = 0;
            *s_token = 0;
            *s_fail = 0;
        }
        __syncthreads();
    }
    if (C > 1) cluster_arrive();  // peers must be running before their mailboxes are written

    RngWords rng;
    {
        const uint4* st = reinterpret_cast<const uint4*>(p.states + (long long)b * RS_STATE_BYTES);
        rng.ctr = st[0]; rng.block = st[1]; rng.key_pos = st[2];
    }
    uint32_t rnd4[4], r0, r1;
    rng_peek2(rng, r0, r1, rnd4);
    const float ux = u01(r0), uy = u01(r1);

    if (bulk_load) {
        if (!mbar_wait_bounded(smem_addr(mbar), 0, p.wait_polls)) wait_failed();
    }

    stamp(1);   // row resident
    // ---- pass 1: x = sanitised scaled logit (sampling.cu:208-227, :547-559); row max; and this
    // thread's own maximum, from which a lower bound for the cutoff is derived below -------------
    float tmax = -INFINITY;
    if (rep) {
#pragma unroll 8
        for (int s = 0; s < Kt; s++) {
            float4 v = bulk_load ? row.ld(s) : ldrow4(s * kLanes + tg);
            const float4 q4 = __ldcg(reinterpret_cast<const float4*>(prow) + s * kLanes + tg);
            v = scaled4_rep(v, q4, a_scale);
            tmax = fmaxf(fmaxf(fmaxf(tmax, v.x), fmaxf(v.y, v.z)), v.w);
            if (SMEM) row.st(s, v);
        }
    } else {
        int s = 0;
        if (SMEM) {
            // Eight groups at a time with ONE test for Inf / NaN products per batch (x * 0 is NaN exactly for those): a
            // branch per group would end the basic block there and leave a lone warp waiting out every instruction.
            for (; s + 8 <= Kt; s += 8) {
                float4 v[8];
                float pr[8], tm = tmax;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float4 l = bulk_load ? row.ld(s + j) : ldrow4((s + j) * kLanes + tg);
                    v[j] = make_float4(l.x * a_scale, l.y * a_scale, l.z * a_scale, l.w * a_scale);
                    pr[j] = fmaf(v[j].w, 0.f, fmaf(v[j].z, 0.f, fmaf(v[j].y, 0.f, v[j].x * 0.f)));
                    tm = fmaxf(fmaxf(fmaxf(tm, v[j].x), fmaxf(v[j].y, v[j].z)), v[j].w);
                }
                const float probe = ((pr[0] + pr[1]) + (pr[2] + pr[3])) + ((pr[4] + pr[5]) + (pr[6] + pr[7]));
                if (probe != probe) {
                    tm = tmax;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        v[j] = sanitize4(v[j]);
                        tm = fmaxf(fmaxf(fmaxf(tm, v[j].x), fmaxf(v[j].y, v[j].z)), v[j].w);
                    }
                }
                tmax = tm;
#pragma unroll
                for (int j = 0; j < 8; j++) row.st(s + j, v[j]);
            }
        }
#pragma unroll 8
        for (; s < Kt; s++) {
            float4 v = bulk_load ? row.ld(s) : ldrow4(s * kLanes + tg);
            v = scaled4(v, a_scale);
            tmax = fmaxf(fmaxf(fmaxf(tmax, v.x), fmaxf(v.y, v.z)), v.w);
            if (SMEM) row.st(s, v);
        }
    }
    stamp(2);   // pass 1 done
    float mx = warp_max(tmax);
    // The warp's sel_rank-th largest thread maximum: at least sel_rank elements of this warp are >= it.
    float wsel = INFINITY;
    const int sel_rank = a_sel_rank;
    if (sel_rank > 0) {
        int rank = 0;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            const float o = __shfl_sync(FULL, tmax, i);
            rank += (o > tmax || (o == tmax && i < lane)) ? 1 : 0;
        }
        const unsigned m = __ballot_sync(FULL, rank == sel_rank - 1);
        wsel = __shfl_sync(FULL, tmax, __ffs(m) - 1);
    }
    if (C > 1) cluster_wait();
    float beta_x;
    {
        const uint32_t* box = exchange(Packets<1>(), pick4(__float_as_uint(mx), __float_as_uint(wsel), 0u, 0u), 0u, 0u);
        mx = warp_max(__uint_as_float(bx(box, 0, lane)));
        beta_x = warp_min(__uint_as_float(bx(box, 1, lane)));   // every warp holds >= sel_rank elements >= beta_x
    }
    stamp(3);   // first exchange done
    const bool try_cand = (sel_rank > 0);
    // Candidates are defined in the domain of e = exp2f(x - max): division by the denominator is
    // monotone, so {e >= beta_e} contains every element whose probability exceeds beta_e / denom.
    float beta_e = try_cand ? exp2f(beta_x - mx) : INFINITY;

    // ---- pass 2: e = exp2f(x - max), ordered denominator (sampling.cu:560-572); min/max of e;
    // elements with e >= beta_e are appended, in order, to this lane's candidate list.  When the list
    // looks too thin to settle the cutoff (not more than top_k strictly above the bound, and about less than
    // top_p of the mass), the bound is lowered 16-fold and the pass repeated, at most twice. -----------
    float acc, emin, emax, csum, denom;
    int nc, ns;   // candidates, and those strictly above the bound
    bool cand_ok;
    uint32_t ncand, nstrict;
    const uint32_t* p2box = nullptr;   // the mailbox of the last second pass: word 4 = candidates of each virtual warp
    auto pass2 = [&](const bool last) -> bool {
            acc = 0.f; emin = INFINITY; emax = -INFINITY;
            nc = 0; ns = 0; csum = 0.f;
        auto pass2_slot = [&](float4 v) {
            v.x = exp2f(v.x - mx);
            v.y = exp2f(v.y - mx);
            v.z = exp2f(v.z - mx);
            v.w = exp2f(v.w - mx);
            float em = 0.f;
            em += v.x; em += v.y; em += v.z; em += v.w;
            acc += em;
            const float hi = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
            emin = fminf(fminf(emin, fminf(v.x, v.y)), fminf(v.z, v.w));
            emax = fmaxf(emax, hi);
            if (hi >= beta_e) {
                append_candidates(v, beta_e, cand + t * 4, L * 4, cap, nc, ns);
                csum += (v.x >= beta_e ? v.x : 0.f) + (v.y >= beta_e ? v.y : 0.f) + (v.z >= beta_e ? v.z : 0.f) +
                        (v.w >= beta_e ? v.w : 0.f);
            }
        };
        // Four groups at a time, with ONE test for candidates per batch: a branch per group would end the basic block
        // there and leave a lone warp waiting out every dependent instruction of its group.
        auto pass2_batch = [&](float4 (&v)[4]) {
            float hi4 = 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                v[j].x = exp2f(v[j].x - mx);
                v[j].y = exp2f(v[j].y - mx);
                v[j].z = exp2f(v[j].z - mx);
                v[j].w = exp2f(v[j].w - mx);
                float em = 0.f;
                em += v[j].x; em += v[j].y; em += v[j].z; em += v[j].w;
                acc += em;
                const float lo = fminf(fminf(v[j].x, v[j].y), fminf(v[j].z, v[j].w));
                const float hi = fmaxf(fmaxf(v[j].x, v[j].y), fmaxf(v[j].z, v[j].w));
                emin = fminf(emin, lo);
                emax = fmaxf(emax, hi);
                hi4 = fmaxf(hi4, hi);
            }
            if (hi4 >= beta_e) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float hi = fmaxf(fmaxf(v[j].x, v[j].y), fmaxf(v[j].z, v[j].w));
                    if (hi >= beta_e) {
                        append_candidates(v[j], beta_e, cand + t * 4, L * 4, cap, nc, ns);
                        csum += (v[j].x >= beta_e ? v[j].x : 0.f) + (v[j].y >= beta_e ? v[j].y : 0.f) + (v[j].z >= beta_e ? v[j].z : 0.f) +
                                (v[j].w >= beta_e ? v[j].w : 0.f);
                    }
                }
            }
        };
        if (SMEM) {
            int s = 0;
            for (; s + 4 <= Kt; s += 4) {
                float4 v[4];
#pragma unroll
                for (int j = 0; j < 4; j++) v[j] = row.ld(s + j);
                pass2_batch(v);
            }
            for (; s < Kt; s++) pass2_slot(row.ld(s));
        } else {
            // streaming variant: the loads of a group of slots are issued together, then consumed in order
            if (rep) {
                constexpr int G = 4;
                const float4* q4p = reinterpret_cast<const float4*>(prow) + tg;
                for (int s0 = 0; s0 < Kt; s0 += G) {
                    float4 lb[G], qb[G];
    #pragma unroll
                    for (int j = 0; j < G; j++) {
                        if (s0 + j < Kt) {
                            lb[j] = ldrow4((s0 + j) * kLanes + tg);
                            qb[j] = __ldcg(q4p + (s0 + j) * kLanes);
                        }
                    }
    #pragma unroll
                    for (int j = 0; j < G; j++) {
                        if (s0 + j < Kt) {
                            pass2_slot(scaled4_rep(lb[j], qb[j], a_scale));
                        }
                    }
                }
            } else {
                constexpr int G = 8;
                for (int s0 = 0; s0 < Kt; s0 += G) {
                    float4 lb[G];
    #pragma unroll
                    for (int j = 0; j < G; j++)
                        if (s0 + j < Kt) lb[j] = ldrow4((s0 + j) * kLanes + tg);
    #pragma unroll
                    for (int j = 0; j < G; j++)
                        if (s0 + j < Kt) pass2_slot(scaled4(lb[j], a_scale));
                }
            }
        }
        stamp(4);   // pass 2 done
        acc = warp_tree_sum(acc);
        emin = warp_min(emin);
        emax = warp_max(emax);
        const unsigned overflow = __any_sync(FULL, nc > cap) ? 1u : 0u;
        const uint32_t wnc = __reduce_add_sync(FULL, (uint32_t)nc), wns = __reduce_add_sync(FULL, (uint32_t)ns);
        csum = warp_tree_sum(csum);
        const uint32_t* box = exchange(Packets<2>(), pick4(__float_as_uint(acc), __float_as_uint(emin), __float_as_uint(emax), overflow),
                                       pick4(wnc, wns, __float_as_uint(csum), 0u), 0u);
        p2box = box;
        denom = warp_tree_sum(__uint_as_float(bx(box, 0, lane)));  // tree over the 32 warp partials (sampling.cu:29-33)
        emin = warp_min(__uint_as_float(bx(box, 1, lane)));
        emax = warp_max(__uint_as_float(bx(box, 2, lane)));
        cand_ok = try_cand && (__reduce_add_sync(FULL, bx(box, 3, lane)) == 0u);
        ncand = __reduce_add_sync(FULL, bx(box, 4, lane));
        nstrict = __reduce_add_sync(FULL, bx(box, 5, lane));
        const float cmass = warp_tree_sum(__uint_as_float(bx(box, 6, lane))) / denom;   // any order: a forecast only
        const bool enough = (use_cnt && nstrict > (uint32_t)a_top_k) || cmass > a_top_p * 1.001f;
        return !cand_ok || enough || last || !(beta_e > 0.f);
    };
    if (!pass2(false)) {
        // A flat row: the lowered bound would already admit every element.  Either the whole row fits the
        // candidate buffer (one more pass with no bound at all), or there is no point in trying.
        const bool all_in = beta_e * 0.0625f <= emin;
        if (all_in && V > cap * kLanes) {
            cand_ok = false;
        } else {
            beta_e = all_in ? 0.f : beta_e * 0.0625f;
            if (!pass2(false)) {
                beta_e *= 0.0625f;
                pass2(true);
            }
        }
    }
    // division is monotone, so the row's min/max probability are the quotients of min/max e
    const float pmin = emin / denom, pmax = emax / denom;
    if (p.dbg_probs) {   // test instrumentation: the probabilities of the whole row
        float* dprow = p.dbg_probs + (long long)b * V;
        for (int s = 0; s < Kt; s++) {
            float4 v = xload(s);
            v.x = exp2f(v.x - mx) / denom;
            v.y = exp2f(v.y - mx) / denom;
            v.z = exp2f(v.z - mx) / denom;
            v.w = exp2f(v.w - mx) / denom;
            reinterpret_cast<float4*>(dprow)[s * kLanes + tg] = v;
        }
    }

    stamp(5);   // second exchange done
    // ---- cutoff search (sampling.cu:593-654, :829-878) ---------------------------------------
    const uint32_t top_k = (uint32_t)a_top_k;
    const float top_p = a_top_p;
    uint32_t left = 0, right = 0, rounds = 0, n_eval = 0;
    uint32_t path = 1;
    uint32_t conv_cnt = 0, conv_left_cnt = 0;   // counts at `right` / `left` and ordered mass at `right` on return
    float conv_mass = 0.f;

    // The reference's loop, replayed with the same pivots and the same decisions.  `lane_eval` returns this
    // lane's ordered masses / counts for four pivots over whatever list the caller searches.
    //  * clamp (candidate list only): every probability above beta_p is on the list, so a pivot above beta_p
    //    sees exactly the elements the reference sees.  A pivot u <= beta_p is not evaluated; instead the set
    //    {p > beta_p} is (pivot u*, the next float after beta_p): if it already holds more than top_k elements
    //    or more than top_p mass, so does the larger set {p >= u}, hence the reference's test at u fails and
    //    its carried state keeps the loop going -- all it uses these values for.  Otherwise: not valid.
    //  * bounds (candidate list only): once every element strictly inside (left, right) has one and the same
    //    value v, the remaining rounds need no data: a pivot equal to `left` selects the set of `left`, a pivot
    //    in (left, v] the set {p >= v}, a pivot above v the set of `right`; they are replayed arithmetically.
    auto run_search = [&](auto&& lane_eval, const bool clamp, const uint32_t beta_p, const bool sure_cnt,
                          const uint32_t n_above) -> bool {
        const uint32_t ustar = clamp ? beta_p + 1u : 0u;
        left = __float_as_uint(pmin);
        right = __float_as_uint(pmax) + 1u;
        rounds = 0;
        uint32_t cnt_x = (uint32_t)V, cnt_r = 0u;   // counts at left / at right
        float mass_x = 1.0f, mass_r = 0.f;
        bool frozen = false, valid = true;
        uint32_t v_bits = 0, cnt_v = 0;
        float mass_v = 0.f;
        while (rounds < 64u) {
            const bool go = use_cnt ? (cnt_x > top_k || mass_x > top_p) : (mass_x > top_p);
            if (!(go && left < right - 1u)) break;
            rounds++;
            const uint32_t pz = (left + right) >> 1, py = (left + pz) >> 1, pw = (pz + right) >> 1;
            const uint32_t pv[3] = {py, pz, pw};
            uint32_t cnt[4];
            float mass[4];
            if (clamp && sure_cnt && pw <= beta_p) {
                // All three pivots lie at or below the bound, and more than top_k elements are known to lie
                // strictly above it: every test fails, the lower end moves to the last pivot, no data is needed.
                left = pw;
                cnt_x = n_above;
                mass_x = 0.f;
                continue;
            }
            if (!frozen) {
                n_eval++;
                const float f[4] = {__uint_as_float(max(py, ustar)), __uint_as_float(max(pz, ustar)),
                                    __uint_as_float(max(pw, ustar)), __uint_as_float(max(left + 1u, ustar))};
                float m[4];
                uint32_t c01, c23, mn, mxv, vmin, vmax;
                lane_eval(f, left, right, cnt_x, m, c01, c23, mn, mxv);
                totals(m, c01, c23, mn, mxv, cnt, mass, vmin, vmax);
                if (clamp && left >= beta_p && vmin >= vmax) {   // one distinct value inside (none: vmin > vmax)
                    frozen = true;
                    v_bits = (vmin == vmax) ? vmin : left;
                    cnt_v = cnt[3];      // the set {p >= left + 1} is {p >= v}
                    mass_v = mass[3];
                }
            } else {
#pragma unroll
                for (int i = 0; i < 3; i++) {
                    const bool at_left = (pv[i] == left), le_v = (pv[i] <= v_bits);
                    cnt[i] = at_left ? cnt_x : le_v ? cnt_v : cnt_r;
                    mass[i] = at_left ? mass_x : le_v ? mass_v : mass_r;
                }
            }
            // the three tests and the bracket update, written with selects: this is the critical path of every round
            bool ok[3], bad = false;
#pragma unroll
            for (int i = 0; i < 3; i++) {
                const bool below = clamp && pv[i] <= beta_p;
                const bool exceeds = (use_cnt && cnt[i] > top_k) || mass[i] > top_p;
                const bool pass = (!use_cnt || cnt[i] < top_k) && mass[i] < top_p;
                ok[i] = !below && pass;
                bad = bad || (below && !exceeds);
            }
            if (bad) { valid = false; break; }
            const bool s0 = ok[0], s1 = !s0 && ok[1], s2 = !s0 && !s1 && ok[2];   // none: the bracket's upper part
            const uint32_t nl = s0 ? left : s1 ? py : s2 ? pz : pw;
            const uint32_t nr = s0 ? py : s1 ? pz : s2 ? pw : right;
            const uint32_t ncx = s0 ? cnt_x : s1 ? cnt[0] : s2 ? cnt[1] : cnt[2];
            const float nmx = s0 ? mass_x : s1 ? mass[0] : s2 ? mass[1] : mass[2];
            const uint32_t ncr = s0 ? cnt[0] : s1 ? cnt[1] : s2 ? cnt[2] : cnt_r;
            const float nmr = s0 ? mass[0] : s1 ? mass[1] : s2 ? mass[2] : mass_r;
            left = nl; right = nr; cnt_x = ncx; mass_x = nmx; cnt_r = ncr; mass_r = nmr;
        }
        conv_cnt = cnt_r;
        conv_mass = mass_r;
        conv_left_cnt = cnt_x;
        return valid && (!clamp || left > beta_p);
    };

    float gtp = 0.f;         // this lane's mass above the threshold, its ties with it, its count above
    uint32_t eqk = 0, gtk = 0;
    bool done = false;
    int quick = 0;           // outcome of the one-warp search on integer masses: 0 not settled that way, 1 settled, 2 list too short
    if (cand_ok) {
        // ===== candidate list: a few elements per lane at most =====
        const int m_own = min(nc, cap);
        for (int i = 0; i < m_own; i++) cand_at(i) = cand_at(i) / denom;
        const uint32_t beta_p = __float_as_uint(beta_e / denom);
        auto cand_eval = [&](const float (&f)[4], uint32_t lo, uint32_t hi, uint32_t, float (&m)[4], uint32_t& c01,
                             uint32_t& c23, uint32_t& mn, uint32_t& mxv) {
            m[0] = m[1] = m[2] = m[3] = 0.f;
            c01 = c23 = 0u;
            mn = 0xffffffffu;
            mxv = 0u;
            for (int i = 0; i < m_own; i++) {
                const float q = cand_at(i);
                const uint32_t qb = __float_as_uint(q);
                if (q >= f[0]) { c01 += 1u; m[0] += q; }
                if (q >= f[1]) { c01 += 0x10000u; m[1] += q; }
                if (q >= f[2]) { c23 += 1u; m[2] += q; }
                if (q >= f[3]) { c23 += 0x10000u; m[3] += q; }
                if (qb > lo && qb < hi) { mn = min(mn, qb); mxv = max(mxv, qb); }
            }
        };
        if (p.quick && ncand <= (uint32_t)kQuickCap) {
            // ---- first try: the whole search in one warp of every CTA, on integer masses (quick_search).  Every
            // CTA gets every candidate of the row: entry k of the list is the same element everywhere (the virtual
            // warps before mine, then the lanes before me), pushed to all CTAs with stores that count their bytes on
            // the destination's barrier.  All CTAs reach the same verdict from the same integers. ----
            uint32_t incl = (uint32_t)m_own;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(FULL, incl, o);
                if (lane >= o) incl += v;
            }
            uint32_t at = __reduce_add_sync(FULL, lane < wg ? bx(p2box, 4, lane) : 0u) + incl - (uint32_t)m_own;
            const uint32_t qb = smem_addr(qbar), ql = smem_addr(qlist);
            if (C > 1 && t == 0) mbar_expect_tx(qb, ncand * 8u);
            for (int i = 0; i < m_own; i++, at++) {
                const float q = cand_at(i);
                const uint32_t w0 = __float_as_uint(q), w1 = __float2uint_rn(q * 1073741824.f);
                if (C == 1) {
                    qlist[at] = make_uint2(w0, w1);
                } else {
#pragma unroll
                    for (int r = 0; r < C; r++) st_async_v2(map_to_cta(ql + at * 8u, (uint32_t)r), w0, w1, map_to_cta(qb, (uint32_t)r));
                }
            }
            if (C == 1) __syncthreads();
            if (wl == 0) {
                if (C > 1 && !mbar_wait_bounded(qb, 0u, p.wait_polls)) wait_failed();
                uint32_t fl = 0u, fr = 0u, fn = 0u;
                const int verdict = (*s_fail == 0) ? quick_search<true>(qlist, ncand, lane, cap + 38, use_cnt, top_k, top_p, beta_p, pmin, pmax,
                                                                  (uint32_t)V, fl, fr, fn)
                                                   : 0;
                if (lane == 0) { s_quick[0] = fl; s_quick[1] = fr; s_quick[2] = fn; s_quick[3] = (uint32_t)verdict; }
            }
            __syncthreads();
            quick = (int)s_quick[3];
            if (quick == 1) { left = s_quick[0]; right = s_quick[1]; rounds = s_quick[2]; }
        }
        if (quick == 2) {
            // the list cannot settle the cutoff: the whole row is searched
        } else if (ncand <= 4096u) {
            done = (quick == 1) ? true : run_search(cand_eval, true, beta_p, use_cnt && nstrict > top_k, nstrict);
            if (done) {
                path = 0;
                const float thr = __uint_as_float(left);
                for (int i = 0; i < m_own; i++) {
                    const float q = cand_at(i);
                    if (q == thr) eqk++;
                    if (q > thr) { gtk++; gtp += q; }
                }
            }
        } else {
            // Long lists (flat rows whose lowered bound took in much of the row): the buffer has the slab's
            // [slot][lane] float4 layout, so it is searched like a slab -- vector loads, and elements below
            // `left` dropped in place once the bracket has risen above the bound.
            for (int i = m_own; i < ((m_own + 3) & ~3); i++) cand_at(i) = -1.f;
            Row<C, true> crow;
            crow.slab = reinterpret_cast<float4*>(cand);
            crow.t = t;
            crow.tg = tg;
            int n = m_own;
            uint32_t list_total = ncand, list_left = 0u;
            auto cand_slab_eval = [&](const float (&f)[4], uint32_t lo, uint32_t, uint32_t cnt_lo, float (&m)[4], uint32_t& c01,
                                      uint32_t& c23, uint32_t& mn, uint32_t& mxv) {
                mn = 0u;
                mxv = 1u;   // bounds are not tracked for long lists
                const bool compact = (lo != list_left) && (lo > beta_p) && (cnt_lo * 2u <= list_total);
                if (compact) {
                    slab_pass<C, true, true>(crow, n, f, __uint_as_float(lo), m, c01, c23);
                    list_total = cnt_lo;
                    list_left = lo;
                } else {
                    slab_pass<C, true, false>(crow, n, f, 0.f, m, c01, c23);
                }
            };
            done = run_search(cand_slab_eval, true, beta_p, use_cnt && nstrict > top_k, nstrict);
            if (done) {
                path = 0;
                const float thr = __uint_as_float(left);
                for (int i = 0; i < n; i++) {
                    const float q = cand_at(i);
                    if (q == thr) eqk++;
                    if (q > thr) { gtk++; gtp += q; }
                }
            }
        }
    }
    if (!done && emin == emax) {
        // Every element has the same probability: the reference's loop never starts (left = pmin, right = left + 1),
        // the threshold is that probability and the whole row ties with it.  No pass is needed.
        left = __float_as_uint(pmin);
        right = left + 1u;
        eqk = (uint32_t)(Kt * 4);
    } else if (!done) {
        // ===== whole row: pass 3, p = exp2f(x - max) / denom (sampling.cu:573-590), in place; then the search
        // over every lane's full list, dropping elements below `left` as the bracket rises =====
#pragma unroll (SMEM ? 2 : 4)
        for (int s = 0; s < Kt; s++) {
            float4 v = xload(s);
            v.x = exp2f(v.x - mx) / denom;
            v.y = exp2f(v.y - mx) / denom;
            v.z = exp2f(v.z - mx) / denom;
            v.w = exp2f(v.w - mx) / denom;
            row.st(s, v);
        }
        int n = Kt * 4;                      // live elements of this lane's list
        uint32_t list_total = (uint32_t)V;   // live elements over the whole row
        uint32_t list_left = __float_as_uint(pmin);   // the list holds exactly the elements >= list_left
        auto slab_eval = [&](const float (&f)[4], uint32_t lo, uint32_t, uint32_t cnt_lo, float (&m)[4], uint32_t& c01,
                             uint32_t& c23, uint32_t& mn, uint32_t& mxv) {
            mn = 0u;
            mxv = 1u;   // bounds are not tracked here
            const bool compact = (lo != list_left) && (cnt_lo * 2u <= list_total);
            if (compact) {
                slab_pass<C, SMEM, true>(row, n, f, __uint_as_float(lo), m, c01, c23);
                list_total = cnt_lo;
                list_left = lo;
            } else {
                slab_pass<C, SMEM, false>(row, n, f, 0.f, m, c01, c23);
            }
        };
        run_search(slab_eval, false, 0u, false, 0u);
        // recount at the threshold (sampling.cu:657-680)
        const float thr = __uint_as_float(left);
        const int slots = (n + 3) >> 2;
#pragma unroll 2
        for (int s = 0; s < slots; s++) {
            const float4 v = row.ld(s);
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (e[j] == thr) eqk++;
                if (e[j] > thr) { gtk++; gtp += e[j]; }
            }
        }
    }
    stamp(6);   // search and recount done
    const bool early_exit = left < right - 1u;
    const float thr = __uint_as_float(left);

    // The reference takes the three totals from block scans; lane 31 of a descending-offset scan holds the
    // same tree value as the butterfly, and the warp values are then added in warp order.
    float sgtp;
    uint32_t seqk, sgtk;
    if (path == 0 && !early_exit && quick != 1) {
        // The bracket closed (right == left + 1): the set at `right` is exactly {p > threshold}, and its count
        // and ordered mass were carried along by the search; the ties are the rest of the set at `left`.
        sgtp = conv_mass;
        sgtk = conv_cnt;
        seqk = conv_left_cnt - conv_cnt;
    } else {
        const float m[4] = {gtp, 0.f, 0.f, 0.f};
        uint32_t cnt[4], d0, d1;
        float mass[4];
        totals(m, gtk | (eqk << 16), 0u, 0u, 0u, cnt, mass, d0, d1);
        sgtp = mass[0];
        sgtk = cnt[0];
        seqk = cnt[1];
    }

    // ---- compensation factor for the boundary ties (sampling.cu:690-696, :903-908) -----------
    float comp = 1.0f;
    if (seqk > 0) {
        comp = fminf(sanitize((top_p - sgtp) / (thr * seqk)), comp);
        if (use_cnt) comp = fminf(sanitize(float(top_k - sgtk) / seqk), comp);
        comp = fmaxf(comp, 0.0f);
    }

    // ---- lane pick (sampling.cu:699-723) -----------------------------------------------------
    const float actual_p = gtp + (thr * eqk) * comp;
    const float incl = warp_scan_desc(actual_p, lane);
    const uint32_t* lbox = exchange(Packets<1>(), __float_as_uint(__shfl_sync(FULL, incl, 31)), 0u, 0u);   // word 0: warp total
    float pre_prev = 0.f, sum_p;   // prefix of the warps before mine; total
    int own_w = -1;                // first warp whose inclusive prefix reaches randp
    float randp;
    {
        // sequential prefix over the warp totals (sampling.cu:85-92)
        float pre[kWarps];
        float s0 = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) {
            const float q = __uint_as_float(bx(lbox, 0, w));
            s0 = (w == 0) ? q : s0 + q;
            pre[w] = s0;
        }
        sum_p = s0;
        randp = sum_p * ux;
#pragma unroll
        for (int w = kWarps - 1; w >= 0; w--) {
            if (randp <= pre[w]) own_w = w;
            if (w == wg - 1) pre_prev = pre[w];
        }
    }
    stamp(7);   // totals and lane-pick exchanges done
    const float cumu_p = (wg > 0) ? incl + pre_prev : incl;
    bool u = (randp <= cumu_p);
    bool u_prev = __shfl_up_sync(FULL, u, 1);
    if (lane == 0) u_prev = (wg > 0) ? (randp <= pre_prev) : false;
    // Exactly one lane sees the 0 -> 1 transition (the scan is non-decreasing); with no
    // transition at all the reference keeps its initial value, lane 0.
    const int owner_cta = (own_w < 0) ? 0 : own_w / WPC;
    const bool is_owner = ((int)crank == owner_cta);
    if (u != u_prev) *s_idxt = tg;

    if (crank == 0 && t == 0 && *s_fail == 0) {  // advance the stored RNG state by one 4-word block
        const uint4 nctr = ctr_next(rng.ctr);
        uint4* st = reinterpret_cast<uint4*>(p.states + (long long)b * RS_STATE_BYTES);
        st[0] = nctr;
        st[1] = philox4x32_10(nctr, rng.key_pos.x, rng.key_pos.y);
    }

    // ---- element pick inside the chosen lane (sampling.cu:725-751), owner CTA only -----------
    int token = -1;
    if (is_owner) {
        __syncthreads();
        const int idxt = *s_idxt;
        float oincl[C];
        int idn_of[C];
#pragma unroll
        for (int it = 0; it < C; it++) {
            const int vt = it * L + t;  // thread index of the reference block
            const int idn = idxt * 4 + (vt >> 2) * 4 * kLanes + (vt & 3);
            float o0 = 0.f;
            if (idn < V) {
                const float x = scaled_logit(ldrow1(idn), rep ? prow[idn] : 0.f, rep, a_scale);
                o0 = exp2f(x - mx) / denom;
            }
            const float o = (o0 < thr) ? 0.f : (o0 == thr) ? (o0 * comp) : o0;
            oincl[it] = warp_scan_desc(o, lane);
            idn_of[it] = idn;
            if (lane == 31) s_wtot[vt >> 5] = oincl[it];
        }
        __syncthreads();
        float opre[C];
        float s0 = 0.f;
#pragma unroll
        for (int it = 0; it < C; it++) opre[it] = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) {
            s0 = (w == 0) ? s_wtot[0] : s0 + s_wtot[w];
#pragma unroll
            for (int it = 0; it < C; it++)
                if (w == it * WPC + wl - 1) opre[it] = s0;
        }
        const float sum_o = s0;
        const float rand2 = sum_o * uy;
#pragma unroll
        for (int it = 0; it < C; it++) {
            const int vw = it * WPC + wl;
            const float cumu_o = (vw > 0) ? oincl[it] + opre[it] : oincl[it];
            const bool uo = (rand2 <= cumu_o);
            bool uo_prev = __shfl_up_sync(FULL, uo, 1);
            if (lane == 0) uo_prev = (vw > 0) ? (rand2 <= opre[it]) : false;
            if (uo != uo_prev) *s_token = (idn_of[it] < V) ? idn_of[it] : 0;
        }
        __syncthreads();
        token = (*s_fail == 0) ? *s_token : -1;
        stamp(8);   // element pick done
        if (t == 0) {
            p.out[b] = token;
            if (ROWP) {
                if (p.out_prob) {   // the sampled id's probability under the full softmax, as the passes computed it
                    float pr = 0.f;
                    if (token >= 0) {
                        const float x = scaled_logit(ldrow1(token), rep ? prow[token] : 0.f, rep, a_scale);
                        pr = exp2f(x - mx) / denom;
                    }
                    p.out_prob[b] = pr;
                }
                if (p.out_kept) p.out_kept[b] = sum_p;
            }
            if (p.dbg_trace) {
                rs_trace tr;
                tr.maxu = mx; tr.denom = denom; tr.pmin = pmin; tr.pmax = pmax; tr.threshold = thr; tr.comp = comp;
                tr.sgtp = sgtp; tr.sum_p = sum_p; tr.randp = randp; tr.sum_o = sum_o; tr.rand2 = rand2;
                tr.left = left; tr.seqk = seqk; tr.sgtk = sgtk; tr.rounds = rounds; tr.idxt = (uint32_t)idxt;
                tr.early_exit = early_exit ? 1u : 0u;
                tr.rnd[0] = rnd4[0]; tr.rnd[1] = rnd4[1]; tr.rnd[2] = rnd4[2]; tr.rnd[3] = rnd4[3];
                tr.token = token;
                tr.path = path;
                tr.ncand = ncand;
#pragma unroll
                for (int i = 0; i < 10; i++) tr.t_ns[i] = ts[i];
                tr.t_ns[0] = n_eval | ((uint32_t)quick << 16);
                p.dbg_trace[b] = tr;
            }
        }
        // out_prob reads the sampled id's OLD penalty: every thread of this CTA stays out of the update until it is read
        if (ROWP && rep && p.out_prob) __syncthreads();
    }

    // ---- penalties: decay everything, add the hit on the sampled id (sampling.cu:427-437).
    // The sampled id lies in the owner CTA's own stripes, so no cross-CTA hand-off is needed. ---
    if (rep && *s_fail == 0) {
#pragma unroll 4
        for (int s = 0; s < Kt; s++) {
            const int i4 = s * kLanes + tg;
            float4 q4 = __ldcg(reinterpret_cast<const float4*>(prow) + i4);
            float e[4] = {q4.x, q4.y, q4.z, q4.w};
            if (i4 != (token >> 2)) {   // token is -1 outside the owner CTA: no group matches
#pragma unroll
                for (int j = 0; j < 4; j++) e[j] = fmaf(e[j], p.decay, 0.f);
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float old = e[j];
                    e[j] = fmaf(old, p.decay, (i4 * 4 + j != token) ? 0.f : (old == 0.f ? p.presence : p.repetition));
                }
            }
            reinterpret_cast<float4*>(prow)[i4] = make_float4(e[0], e[1], e[2], e[3]);
        }
    }
}

__global__ void setup_rand_kernel(unsigned char* states, unsigned long long seed, long long B, long long first_row) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B) return;
    const unsigned long long sub = (unsigned long long)(first_row + i);
    const uint4 ctr = make_uint4(0u, 0u, (uint32_t)sub, (uint32_t)(sub >> 32));
    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    uint4* st = reinterpret_cast<uint4*>(states + i * RS_STATE_BYTES);
    st[0] = ctr;
    st[1] = philox4x32_10(ctr, k0, k1);
    st[2] = make_uint4(k0, k1, 0u, 0u);
    st[3] = make_uint4(0u, 0u, 0u, 0u);
}

// Test instrumentation for the failure path: one CTA waits, with the given poll limit, on an mbarrier that nothing
// will ever complete, and reports the expiry exactly as the sampler does.  No copy or remote store is in flight,
// so nothing can land in the shared memory of the CTA after it has returned.
__global__ void selftest_wait_kernel(int* status, int* status_mirror, uint32_t polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_addr(&bar), 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait_bounded(smem_addr(&bar), 0, polls)) {
        atomicExch(status, RS_ERR_TIMEOUT);
        if (status_mirror) *reinterpret_cast<volatile int*>(status_mirror) = RS_ERR_TIMEOUT;
    }
}

// Per-row parameters: the host functions' checks and remaps (sampling.cu:458-486, :982-1011) applied to every row
// on the device.  A temperature outside [0.001, 1000] cannot raise here; the row is sampled at temperature 1 and
// the status word reports RS_ERR_TEMPERATURE.
__global__ void row_args_kernel(int B, int V, const float* temperature, const int* top_k, const float* top_p, int rep,
                                int allow_candidates, RowArgs* out, int* status, int* status_mirror) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    float tmp = temperature ? temperature[b] : 1.0f;
    long long k = top_k ? top_k[b] : -1;
    float pp = top_p ? top_p[b] : 1.0f;
    if (!(tmp >= 0.001f && tmp <= 1000.f)) {
        atomicExch(status, RS_ERR_TEMPERATURE);
        if (status_mirror) *reinterpret_cast<volatile int*>(status_mirror) = RS_ERR_TEMPERATURE;
        tmp = 1.0f;
    }
    if (k <= 0 || k > V) k = V;
    if (pp < 0.f || pp > 1.f || pp != pp) pp = 1.f;
    if (pp == 0.f) { k = 1; pp = 1.f; }
    RowArgs r;
    r.kind = rep ? kRepetition : ((tmp == 1.0f && k == V) ? kTopP : kGeneral);
    r.top_k = (int)k;
    r.top_p = pp;
    r.scale = (r.kind == kTopP) ? (float)1.4426950408889634074 : (float)(1.4426950408889634074 / (double)tmp);
    // rank of the thread maximum that bounds the candidate list: same rule as for per-call parameters
    int sel = 0;
    if (allow_candidates && !(k >= V && pp >= 1.0f)) {
        if (k < V) sel = (k + 2 > 256) ? 0 : (int)((k + 2 + 31) / 32);
        else sel = 2;
    }
    r.sel_rank = sel;
    r.pad0 = 0; r.pad1 = r.pad2 = 0.f;
    out[b] = r;
}

// ------------------------------------------------------------------ host side -------------
struct DeviceInfo {
    bool ready = false;
    int sms = 0, smem_optin = 0, smem_sm = 0;
    bool attr_set[20][3] = {};
    int* mirror = nullptr;   // host word the kernels copy a non-zero status to (rs_set_status_mirror)
};
static DeviceInfo g_dev[64];
static std::mutex g_mu;
static std::atomic<uint64_t> g_launches{0};
static std::atomic<int> g_cluster_override{0};
static std::atomic<int> g_path_override{0};
static std::atomic<uint32_t> g_wait_polls{kDefaultWaitPolls};
static std::atomic<int> g_dependent_launch{1};   // sampler kernels are launched with programmatic stream serialization
constexpr long long kRowCtaMinBatch = 112;   // from here on one CTA per row (two rows per SM beyond 148 rows) beats the cluster variants
static thread_local char g_err[256] = "";

static int cuda_fail(cudaError_t e, const char* what) {
    snprintf(g_err, sizeof g_err, "%s: %s", what, cudaGetErrorString(e));
    return RS_ERR_CUDA;
}

static int cidx(int C) { return C == 1 ? 0 : C == 2 ? 1 : C == 4 ? 2 : C == 8 ? 3 : 4; }

template <int C, bool SMEM, bool LOWP, bool ROWP = false, bool MORE_REGS = false>
static int launch_typed(const Params& p, int smem, cudaStream_t stream, DeviceInfo& di) {
    if constexpr (!SMEM && C == 8 && !MORE_REGS) {
        // batches whose CTAs all fit at 6 per SM take the instantiation with more registers (C3: 32.0 -> 30.4 us,
        // C5: 316 -> 290 us); larger ones need the 8 CTAs per SM of the 64-register one
        if ((long long)p.B * C <= (long long)di.sms * 6) return launch_typed<C, SMEM, LOWP, ROWP, true>(p, smem, stream, di);
    }
    auto kern = sampler_kernel<C, SMEM, LOWP, ROWP, MORE_REGS>;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!di.attr_set[cidx(C) + (LOWP ? 5 : 0) + (ROWP ? 10 : 0)][SMEM ? 1 : (MORE_REGS ? 2 : 0)]) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di.smem_optin);
            if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(smem)");
            if (C > 8) {
                e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
                if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(cluster)");
            }
            di.attr_set[cidx(C) + (LOWP ? 5 : 0) + (ROWP ? 10 : 0)][SMEM ? 1 : (MORE_REGS ? 2 : 0)] = true;
        }
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3((unsigned)(p.B * C), 1, 1);
    cfg.blockDim = dim3(kLanes / C, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    int na = 0;
    if (C > 1) {
        at[na].id = cudaLaunchAttributeClusterDimension;
        at[na].val.clusterDim.x = C;
        at[na].val.clusterDim.y = 1;
        at[na].val.clusterDim.z = 1;
        na++;
    }
    // Early scheduling pays for small grids (measured: B=1 24.7 -> 23.1 us, B=4 53.2 -> 51.3 us per back-to-back call).  A
    // grid that fills most of the GPU is better placed on an empty one: its CTAs would take whatever slots the
    // predecessor left free and end up unevenly spread (B=64, 512 CTAs: 36.6 -> 39.9 us).
    if (g_dependent_launch.load() && (long long)p.B * C * 2 <= di.sms) {   // the kernel waits for its predecessor itself
        at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = at;
    cfg.numAttrs = (unsigned)na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(sampler)");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return RS_OK;
}

template <int C, bool SMEM>
static int launch_one(const Params& p, int smem, cudaStream_t stream, DeviceInfo& di) {
    return p.dtype == RS_DTYPE_F32 ? launch_typed<C, SMEM, false>(p, smem, stream, di)
                                   : launch_typed<C, SMEM, true>(p, smem, stream, di);
}
// per-row parameters: the widths the planner picks by itself (8 or 16 CTAs on chip, 8 streaming)
template <int C, bool SMEM>
static int launch_rows(const Params& p, int smem, cudaStream_t stream, DeviceInfo& di) {
    return p.dtype == RS_DTYPE_F32 ? launch_typed<C, SMEM, false, true>(p, smem, stream, di)
                                   : launch_typed<C, SMEM, true, true>(p, smem, stream, di);
}

static int get_device(DeviceInfo** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return RS_ERR_LIMIT;
    DeviceInfo& di = g_dev[dev];
    std::lock_guard<std::mutex> lk(g_mu);
    if (!di.ready) {
        if ((e = cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return cuda_fail(e, "attr");
        if ((e = cudaDeviceGetAttribute(&di.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return cuda_fail(e, "attr");
        if ((e = cudaDeviceGetAttribute(&di.smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev)) != cudaSuccess) return cuda_fail(e, "attr");
        di.ready = true;
    }
    *out = &di;
    return RS_OK;
}

// Rank of the per-warp thread maximum used as the lower bound of the candidate shortcut, and the
// candidate buffer's float4 slots per lane.  With rank j every warp holds >= j elements above the
// bound, 32*j in the row: enough to exceed top_k.  Without a usable top_k the loosest bound (the
// smallest thread maximum) is tried and the kernel checks the mass condition itself.
static void choose_candidates(long long V, long long top_k, double top_p, int* sel_rank, int* cand_slots) {
    *sel_rank = 0;
    *cand_slots = 0;
    if (g_path_override.load() == 1) return;
    if (top_k >= V && top_p >= 1.0) return;            // nothing is filtered: the whole row is kept
    // Beyond top_k ~ 250 the candidate lists stop being short; such calls search the whole row.
    if (top_k < V) {
        if (top_k + 2 > 256) return;
        *sel_rank = (int)((top_k + 2 + 31) / 32);
    } else {
        *sel_rank = 2;                                  // top-p only: try the ~200 largest; the kernel checks their mass
    }
    *cand_slots = (*sel_rank <= 4) ? 2 : 4;
}

static int smem_need(int V, int C, int cand_slots) { return kSlabOff + cand_slots * (kLanes / C) * 16 + slab_bytes(V, C); }

// Which kernel variant serves a call.
//  * on-chip: the row stays in the cluster's shared memory (one HBM read, lowest latency).  Used while the
//    whole batch is resident at once; beyond that rows would queue for shared memory.
//  * streaming: nothing but the candidate lists is kept on chip; the row is read twice (the second time from
//    L2), any number of rows is in flight, and a row whose candidates do not settle the cutoff falls back to a
//    global scratch row (the counterpart of the reference's `probs`, sampling.cu:488).  Needs B*V floats.
struct Plan {
    int C;
    bool smem;
    bool rowcta;       // one CTA per row with several virtual lanes per thread (rs_rowcta.cu): large batches
    int sel_rank, cand_slots;
    size_t ws;
};
static size_t ws_bytes(long long B, long long V) { return 256 + (size_t)B * (size_t)V * sizeof(float); }

static Plan make_plan(const DeviceInfo& di, long long B, int V, int sel_rank, int cand_slots, size_t ws_avail) {
    Plan pl;
    pl.rowcta = false;
    pl.sel_rank = sel_rank;
    pl.cand_slots = cand_slots;
    auto fits = [&](int C) { return smem_need(V, C, cand_slots) <= di.smem_optin; };
    auto resident_rows = [&](int C) {
        const int need = smem_need(V, C, cand_slots) + 1024;
        int per_sm = di.smem_sm / need;
        per_sm = per_sm < 2048 / (kLanes / C) ? per_sm : 2048 / (kLanes / C);
        per_sm = per_sm < ctas_per_sm_by_registers(C, true) ? per_sm : ctas_per_sm_by_registers(C, true);
        if (per_sm > 32) per_sm = 32;
        return (long long)di.sms * per_sm / C;
    };
    const int forced = g_cluster_override.load();
    const int mode = g_path_override.load();
    const bool can_stream = ws_avail >= ws_bytes(B, V);
    // the streaming variant has shared memory to spare: room for 32 candidates per lane, so that lowered bounds fit
    auto streaming = [&]() { pl.C = 8; pl.smem = false; pl.ws = ws_bytes(B, V); if (pl.cand_slots) pl.cand_slots = 8; return pl; };
    auto onchip = [&](int C) { pl.C = C; pl.smem = true; pl.ws = 256; return pl; };
    if (forced) return fits(forced) ? onchip(forced) : streaming();
    if (mode == 2) return streaming();
    if (fits(8) && (B <= resident_rows(8) || mode == 3 || !can_stream)) return onchip(8);
    if (!fits(8) && fits(16) && (B <= resident_rows(16) || mode == 3 || !can_stream)) return onchip(16);
    return streaming();
}

static int sample_impl(const void* logits, int dtype, int64_t B, int64_t T, int64_t V, float* penalties, void* states, int32_t* out,
                       double temperature, int64_t top_k, double top_p, double presence, double repetition, double decay,
                       void* workspace, size_t workspace_bytes, void* stream, float* dbg_probs, rs_trace* dbg_trace) {
    // checks and remaps of the reference's host functions (sampling.cu:458-486, :982-1011)
    if (!(V > 0 && V <= 1048576 && V % 4 == 0)) return RS_ERR_VOCAB;
    if (!(B > 0 && T > 0)) return RS_ERR_BATCH;
    if (!(temperature >= 0.001 && temperature <= 1000)) return RS_ERR_TEMPERATURE;
    if (B > (1ll << 24)) return RS_ERR_LIMIT;
    if (dtype != RS_DTYPE_F32 && dtype != RS_DTYPE_F16 && dtype != RS_DTYPE_BF16) return RS_ERR_DTYPE;
    if (!logits || !states || !out || !workspace) return RS_ERR_POINTER;
    if (((uintptr_t)logits & (dtype == RS_DTYPE_F32 ? 15 : 7)) || ((uintptr_t)states & 15) || ((uintptr_t)penalties & 15) ||
        ((uintptr_t)workspace & 255))
        return RS_ERR_POINTER;
    if (top_k <= 0 || top_k > V) top_k = V;
    if (top_p < 0 || top_p > 1) top_p = 1;
    if (top_p == 0) { top_k = 1; top_p = 1; }
    const double log2e_inv_temp = 1.4426950408889634074 / temperature;

    DeviceInfo* di = nullptr;
    int rc = get_device(&di);
    if (rc) return rc;
    int sel_rank = 0, cand_slots = 0;
    choose_candidates(V, top_k, top_p, &sel_rank, &cand_slots);
    Plan pl = make_plan(*di, B, (int)V, sel_rank, cand_slots, workspace_bytes);
    // Large batches: one CTA per row, several rows per SM.  Needs the scratch rows for its whole-row fallback.
    {
        const int mode = g_path_override.load();
        const bool eligible = workspace_bytes >= ws_bytes(B, V);
        // A call that is known to search the whole row -- a top_k too large for the candidate bound, or no cutoff at
        // all -- stays with the cluster kernel: 1024 threads per row carry the full-row rounds better than 256.  So
        // does a call without a top_k whose top_p is large: its kept set may be a good part of the row (N(0, 3^2)
        // logits: 4 % at top_p 0.9), which overflows this kernel's 6 entries per lane but not the cluster kernel's 32.
        const bool wide = V > 8192 && (sel_rank == 0 || (top_k == V && top_p > 0.5));   // (short rows: a whole-row search is cheap)
        const bool wanted = (mode == 4 || mode == 5) ||
                            ((mode == 0 || mode == 6) && g_cluster_override.load() == 0 && !pl.smem && B >= kRowCtaMinBatch && !wide);
        if (eligible && wanted) {
            pl.rowcta = true;
            pl.ws = ws_bytes(B, V);
        }
    }
    if (workspace_bytes < pl.ws) return RS_ERR_WORKSPACE;
    const bool use_smem = pl.smem;
    const int C = pl.C;
    cand_slots = pl.cand_slots;

    Params p;
    p.logits = (const char*)logits + (T - 1) * V * (dtype == RS_DTYPE_F32 ? 4 : 2);
    p.dtype = dtype;
    p.row_stride = (long long)T * V;
    p.penalties = penalties;
    p.states = (unsigned char*)states;
    p.out = out;
    p.status = (int*)workspace;
    p.status_mirror = di->mirror;
    p.wait_polls = g_wait_polls.load();
    p.scratch = (float*)((char*)workspace + 256);
    p.dbg_probs = dbg_probs;
    p.dbg_trace = dbg_trace;
    p.rows = nullptr;
    p.out_prob = nullptr;
    p.out_kept = nullptr;
    p.quick = (g_path_override.load() < 5) ? 1 : 0;
    p.B = (int)B;
    p.V = (int)V;
    p.kind = penalties ? kRepetition : ((temperature == 1 && top_k == V) ? kTopP : kGeneral);
    p.top_k = (int)top_k;
    p.scale = (p.kind == kTopP) ? (float)1.4426950408889634074 : (float)log2e_inv_temp;
    p.top_p = (float)top_p;
    p.presence = (float)presence;
    p.repetition = (float)repetition;
    p.decay = (float)decay;
    p.sel_rank = sel_rank;
    p.cand_slots = cand_slots;

    cudaStream_t st = (cudaStream_t)stream;
    if (pl.rowcta) {
        // up to 148 rows: one CTA per SM with all of its shared memory; more: two CTAs share an SM
        const int budget = (B <= di->sms) ? di->smem_optin : (di->smem_sm / 2 - 1024);
        const int lpt = (B <= di->sms) ? 2 : 4;
        const RowCtaPlan rp = rowcta_plan((int)V, penalties != nullptr, sel_rank, lpt, budget);
        rc = rowcta_launch(p, rp, lpt, st, di->smem_optin, g_dependent_launch.load() != 0 && B * 2 <= di->sms);
        if (rc == RS_OK) g_launches.fetch_add(1, std::memory_order_relaxed);
        else if (rc == RS_ERR_CUDA) return cuda_fail(cudaGetLastError(), "launch(rowcta)");
        return rc;
    }
    if (!use_smem) return launch_one<8, false>(p, kSlabOff + cand_slots * (kLanes / 8) * 16, st, *di);
    const int smem = smem_need((int)V, C, cand_slots);
    switch (C) {
        case 1: return launch_one<1, true>(p, smem, st, *di);
        case 2: return launch_one<2, true>(p, smem, st, *di);
        case 4: return launch_one<4, true>(p, smem, st, *di);
        case 8: return launch_one<8, true>(p, smem, st, *di);
        case 16: return launch_one<16, true>(p, smem, st, *di);
    }
    return RS_ERR_LIMIT;
}


// Per-row temperature / top_k / top_p (device arrays of B values; a null array means the neutral value for every
// row: temperature 1, top_k -1, top_p 1).  Workspace: 256 B status, the rows' normalised parameters, then the
// scratch rows of the streaming variant.
static size_t row_args_bytes(long long B) { return ((size_t)B * sizeof(RowArgs) + 255) & ~(size_t)255; }

static int sample_rows_impl(const void* logits, int dtype, int64_t B, int64_t T, int64_t V, float* penalties, void* states,
                            int32_t* out, const float* temperature, const int32_t* top_k, const float* top_p, double presence,
                            double repetition, double decay, float* out_prob, float* out_kept, void* workspace,
                            size_t workspace_bytes, void* stream) {
    if (!(V > 0 && V <= 1048576 && V % 4 == 0)) return RS_ERR_VOCAB;
    if (!(B > 0 && T > 0)) return RS_ERR_BATCH;
    if (B > (1ll << 24)) return RS_ERR_LIMIT;
    if (dtype != RS_DTYPE_F32 && dtype != RS_DTYPE_F16 && dtype != RS_DTYPE_BF16) return RS_ERR_DTYPE;
    if (!logits || !states || !out || !workspace) return RS_ERR_POINTER;
    if (((uintptr_t)logits & (dtype == RS_DTYPE_F32 ? 15 : 7)) || ((uintptr_t)states & 15) || ((uintptr_t)penalties & 15) ||
        ((uintptr_t)workspace & 255) || ((uintptr_t)temperature & 3) || ((uintptr_t)top_k & 3) || ((uintptr_t)top_p & 3))
        return RS_ERR_POINTER;
    DeviceInfo* di = nullptr;
    int rc = get_device(&di);
    if (rc) return rc;
    const size_t rab = row_args_bytes(B);
    if (workspace_bytes < 256 + rab) return RS_ERR_WORKSPACE;
    // rows differ in top_k: the candidate buffer takes the widest size
    const bool allow_cand = g_path_override.load() != 1;
    Plan pl = make_plan(*di, B, (int)V, allow_cand ? 8 : 0, allow_cand ? 4 : 0, workspace_bytes - rab);
    {   // large batches: one CTA per row, as for per-call parameters
        const int mode = g_path_override.load();
        const bool eligible = workspace_bytes - rab >= ws_bytes(B, V);
        const bool wanted = (mode == 4 || mode == 5) || ((mode == 0 || mode == 6) && g_cluster_override.load() == 0 && !pl.smem && B >= kRowCtaMinBatch);
        if (eligible && wanted) {
            pl.rowcta = true;
            pl.ws = ws_bytes(B, V);
        }
    }
    if (workspace_bytes < pl.ws + rab) return RS_ERR_WORKSPACE;
    if (pl.smem && pl.C != 8 && pl.C != 16) return RS_ERR_LIMIT;   // forced widths exist for the per-call entry only

    cudaStream_t st = (cudaStream_t)stream;
    RowArgs* rows = (RowArgs*)((char*)workspace + 256);
    row_args_kernel<<<(unsigned)((B + 127) / 128), 128, 0, st>>>((int)B, (int)V, temperature, top_k, top_p, penalties ? 1 : 0,
                                                               allow_cand ? 1 : 0, rows, (int*)workspace, di->mirror);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "launch(row_args)");
    g_launches.fetch_add(1, std::memory_order_relaxed);

    Params p;
    p.logits = (const char*)logits + (T - 1) * V * (dtype == RS_DTYPE_F32 ? 4 : 2);
    p.dtype = dtype;
    p.row_stride = (long long)T * V;
    p.penalties = penalties;
    p.states = (unsigned char*)states;
    p.out = out;
    p.status = (int*)workspace;
    p.status_mirror = di->mirror;
    p.wait_polls = g_wait_polls.load();
    p.scratch = (float*)((char*)workspace + 256 + rab);
    p.dbg_probs = nullptr;
    p.dbg_trace = nullptr;
    p.rows = rows;
    p.out_prob = out_prob;
    p.out_kept = out_kept;
    p.quick = (g_path_override.load() < 5) ? 1 : 0;
    p.B = (int)B;
    p.V = (int)V;
    p.kind = penalties ? kRepetition : kGeneral;   // the kernel takes kind, top_k, top_p, scale and the rank from `rows`
    p.top_k = (int)V;
    p.scale = 1.f;
    p.top_p = 1.f;
    p.presence = (float)presence;
    p.repetition = (float)repetition;
    p.decay = (float)decay;
    p.sel_rank = 0;
    p.cand_slots = pl.cand_slots;
    if (pl.rowcta) {
        const int budget = (B <= di->sms) ? di->smem_optin : (di->smem_sm / 2 - 1024);
        const int lpt = (B <= di->sms) ? 2 : 4;
        const RowCtaPlan rp = rowcta_plan((int)V, penalties != nullptr, allow_cand ? 8 : 0, lpt, budget);
        rc = rowcta_launch(p, rp, lpt, st, di->smem_optin, g_dependent_launch.load() != 0 && B * 2 <= di->sms);
        if (rc == RS_OK) g_launches.fetch_add(1, std::memory_order_relaxed);
        else if (rc == RS_ERR_CUDA) return cuda_fail(cudaGetLastError(), "launch(rowcta, per-row)");
        return rc;
    }
    if (!pl.smem) return launch_rows<8, false>(p, kSlabOff + pl.cand_slots * (kLanes / 8) * 16, st, *di);
    const int smem = smem_need((int)V, pl.C, pl.cand_slots);
    return pl.C == 8 ? launch_rows<8, true>(p, smem, st, *di) : launch_rows<16, true>(p, smem, st, *di);
}


// ---------------------------------------------------------------------------------------------
// Scratch that lives inside the library image, for rs_sample_static_scratch().
//
// Some hosts may not allocate device memory when they want to sample: a serving process that has
// handed all of HBM to its own arena at start-up has nothing left for cudaMalloc to give, and a
// latency-critical decode loop must not call an allocator that can synchronise the whole device.
// For them the global-scratch-row variant of the sampler runs on this fixed array instead of a
// caller-provided workspace.  Layout: 256 bytes of status word, then the scratch rows.
// Every GPU that loads the library carries the array (16 MiB + 256 B) until the process exits.
static __device__ __align__(256) float g_static_scratch[64 + RS_STATIC_SCRATCH_FLOATS];
static float* g_static_ptr[64] = {};   // device address of the array, per device, filled at set-up

// Set-up, once per device, with that device current.  In host code the array's NAME is only a
// host-side handle; the device address has to be asked for.
static int static_scratch_address(int dev, cudaStream_t stream, float** out) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_static_ptr[dev]) {
        float* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        if (!ptr) return RS_ERR_POINTER;
        // the status word starts clear (on the caller's stream, ahead of the first launch); the rows need no
        // clearing: the kernel writes them before it reads them
        e = cudaMemsetAsync(ptr, 0, 256, stream);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(static status word)");
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return RS_OK;
}

static int sample_static_impl(const float* logits, int64_t B, int64_t T, int64_t V, float* penalties, void* states,
                              int32_t* out, double temperature, int64_t top_k, double top_p, double presence,
                              double repetition, double decay, void* stream) {
    if (!(V > 0 && V <= 1048576 && V % 4 == 0)) return RS_ERR_VOCAB;
    if (!(B > 0 && T > 0)) return RS_ERR_BATCH;
    if (!(temperature >= 0.001 && temperature <= 1000)) return RS_ERR_TEMPERATURE;
    if (B > (int64_t)RS_STATIC_SCRATCH_FLOATS / V) return RS_ERR_LIMIT;   // B * V cannot wrap this way
    if (!logits || !states || !out) return RS_ERR_POINTER;
    if (((uintptr_t)logits & 15) || ((uintptr_t)states & 15) || ((uintptr_t)penalties & 15)) return RS_ERR_POINTER;
    if (top_k <= 0 || top_k > V) top_k = V;
    if (top_p < 0 || top_p > 1) top_p = 1;
    if (top_p == 0) { top_k = 1; top_p = 1; }
    DeviceInfo* di = nullptr;
    int rc = get_device(&di);
    if (rc) return rc;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    float* base = nullptr;
    rc = static_scratch_address(dev, (cudaStream_t)stream, &base);
    if (rc) return rc;
    Params p;
    p.logits = logits + (T - 1) * V;
    p.dtype = RS_DTYPE_F32;
    p.row_stride = (long long)T * V;
    p.penalties = penalties;
    p.states = (unsigned char*)states;
    p.out = out;
    p.status = (int*)base;
    p.status_mirror = di->mirror;
    p.wait_polls = g_wait_polls.load();
    p.scratch = base + 64;
    p.dbg_probs = nullptr;
    p.dbg_trace = nullptr;
    p.rows = nullptr;
    p.out_prob = nullptr;
    p.out_kept = nullptr;
    p.quick = (g_path_override.load() < 5) ? 1 : 0;
    p.B = (int)B;
    p.V = (int)V;
    p.kind = penalties ? kRepetition : ((temperature == 1 && top_k == V) ? kTopP : kGeneral);
    p.top_k = (int)top_k;
    p.scale = (p.kind == kTopP) ? (float)1.4426950408889634074 : (float)(1.4426950408889634074 / temperature);
    p.top_p = (float)top_p;
    p.presence = (float)presence;
    p.repetition = (float)repetition;
    p.decay = (float)decay;
    p.sel_rank = 0;
    p.cand_slots = 0;
    return launch_one<8, false>(p, kSlabOff, (cudaStream_t)stream, *di);
}

}  // namespace rs

// ------------------------------------------------------------------- C ABI -----------------
extern "C" {

int rs_setup_rand(void* states_device, uint64_t seed, int64_t B, int64_t first_row, void* stream) {
    if (B <= 0) return RS_ERR_BATCH;
    if (!states_device || ((uintptr_t)states_device & 15)) return RS_ERR_POINTER;
    const int threads = 128;
    const unsigned blocks = (unsigned)((B + threads - 1) / threads);
    rs::setup_rand_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>((unsigned char*)states_device, seed, B, first_row);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return rs::cuda_fail(e, "setup_rand launch");
    rs::g_launches.fetch_add(1, std::memory_order_relaxed);
    return RS_OK;
}

size_t rs_workspace_bytes(int64_t B, int64_t V) {
    if (B <= 0 || V <= 0 || V > 1048576) return 256;
    rs::DeviceInfo b200;   // the library is built for B200 only: 148 SMs, 227 KiB per CTA, 228 KiB per SM
    b200.sms = 148;
    b200.smem_optin = 232448;
    b200.smem_sm = 233472;
    // sized for the widest candidate buffer, so that any top_k / top_p of a later call is covered
    return rs::make_plan(b200, B, (int)V, 8, 4, ~(size_t)0).ws;
}

int rs_sample(const float* logits_device, int64_t B, int64_t T, int64_t V, float* penalties_device, void* states_device,
              int32_t* out_device, double temperature, int64_t top_k, double top_p, double presence_penalty,
              double repetition_penalty, double penalty_decay, void* workspace_device, size_t workspace_bytes,
              void* stream) {
    return rs::sample_impl(logits_device, RS_DTYPE_F32, B, T, V, penalties_device, states_device, out_device, temperature, top_k, top_p,
                           presence_penalty, repetition_penalty, penalty_decay, workspace_device, workspace_bytes, stream,
                           nullptr, nullptr);
}

int rs_sample_debug(const float* logits_device, int64_t B, int64_t T, int64_t V, float* penalties_device,
                    void* states_device, int32_t* out_device, double temperature, int64_t top_k, double top_p,
                    double presence_penalty, double repetition_penalty, double penalty_decay, void* workspace_device,
                    size_t workspace_bytes, void* stream, float* probs_device, rs_trace* trace_device) {
    return rs::sample_impl(logits_device, RS_DTYPE_F32, B, T, V, penalties_device, states_device, out_device, temperature, top_k, top_p,
                           presence_penalty, repetition_penalty, penalty_decay, workspace_device, workspace_bytes, stream,
                           probs_device, trace_device);
}

int rs_sample_host(const float* logits_host, int64_t B, int64_t T, int64_t V, float* penalties_device,
                   void* states_device, int32_t* out_host, double temperature, int64_t top_k, double top_p,
                   double presence_penalty, double repetition_penalty, double penalty_decay, float* staging_device,
                   int32_t* out_device, void* workspace_device, size_t workspace_bytes, void* stream) {
    if (!logits_host || !out_host || !staging_device || !out_device) return RS_ERR_POINTER;
    if (!(V > 0 && V <= 1048576 && V % 4 == 0)) return RS_ERR_VOCAB;
    if (!(B > 0 && T > 0)) return RS_ERR_BATCH;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (T == 1) {
        e = cudaMemcpyAsync(staging_device, logits_host, (size_t)B * V * sizeof(float), cudaMemcpyHostToDevice, st);
    } else {  // only the last position of every row crosses the bus
        e = cudaMemcpy2DAsync(staging_device, (size_t)V * sizeof(float), logits_host + (T - 1) * V,
                              (size_t)T * V * sizeof(float), (size_t)V * sizeof(float), (size_t)B, cudaMemcpyHostToDevice, st);
    }
    if (e != cudaSuccess) return rs::cuda_fail(e, "logits H2D");
    int rc = rs::sample_impl(staging_device, RS_DTYPE_F32, B, 1, V, penalties_device, states_device, out_device, temperature, top_k,
                             top_p, presence_penalty, repetition_penalty, penalty_decay, workspace_device,
                             workspace_bytes, stream, nullptr, nullptr);
    if (rc) return rc;
    e = cudaMemcpyAsync(out_host, out_device, (size_t)B * sizeof(int32_t), cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return rs::cuda_fail(e, "ids D2H");
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return rs::cuda_fail(e, "cudaStreamSynchronize");
    return RS_OK;
}

int rs_sample_typed(const void* logits_device, int32_t logits_dtype, int64_t B, int64_t T, int64_t V, float* penalties_device,
                    void* states_device, int32_t* out_device, double temperature, int64_t top_k, double top_p,
                    double presence_penalty, double repetition_penalty, double penalty_decay, void* workspace_device,
                    size_t workspace_bytes, void* stream, float* probs_device, rs_trace* trace_device) {
    return rs::sample_impl(logits_device, logits_dtype, B, T, V, penalties_device, states_device, out_device, temperature,
                           top_k, top_p, presence_penalty, repetition_penalty, penalty_decay, workspace_device,
                           workspace_bytes, stream, probs_device, trace_device);
}

size_t rs_rows_workspace_bytes(int64_t B, int64_t V) {
    if (B <= 0) return 256;
    return rs_workspace_bytes(B, V) + rs::row_args_bytes(B);
}

int rs_sample_rows(const void* logits_device, int32_t logits_dtype, int64_t B, int64_t T, int64_t V, float* penalties_device,
                   void* states_device, int32_t* out_device, const float* temperature_device, const int32_t* top_k_device,
                   const float* top_p_device, double presence_penalty, double repetition_penalty, double penalty_decay,
                   float* out_prob_device, float* out_kept_mass_device, void* workspace_device, size_t workspace_bytes,
                   void* stream) {
    return rs::sample_rows_impl(logits_device, logits_dtype, B, T, V, penalties_device, states_device, out_device,
                                temperature_device, top_k_device, top_p_device, presence_penalty, repetition_penalty,
                                penalty_decay, out_prob_device, out_kept_mass_device, workspace_device, workspace_bytes, stream);
}

int rs_device_status(void* workspace_device, void* stream) {
    int v = 0;
    if (!workspace_device) {   // the status word of rs_sample_static_scratch's built-in array on the current device
        int dev = 0;
        cudaError_t e0 = cudaGetDevice(&dev);
        if (e0 != cudaSuccess) return rs::cuda_fail(e0, "cudaGetDevice");
        if (dev < 0 || dev >= 64) return RS_ERR_LIMIT;
        float* base = nullptr;
        const int rc = rs::static_scratch_address(dev, (cudaStream_t)stream, &base);
        if (rc) return rc;
        workspace_device = base;
    }
    cudaError_t e = cudaMemcpyAsync(&v, workspace_device, sizeof v, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return rs::cuda_fail(e, "status read");
    return v;
}

int rs_clear_status(void* workspace_device, void* stream) {
    if (!workspace_device) {
        int dev = 0;
        cudaError_t e0 = cudaGetDevice(&dev);
        if (e0 != cudaSuccess) return rs::cuda_fail(e0, "cudaGetDevice");
        if (dev < 0 || dev >= 64) return RS_ERR_LIMIT;
        float* base = nullptr;
        const int rc = rs::static_scratch_address(dev, (cudaStream_t)stream, &base);
        if (rc) return rc;
        workspace_device = base;
    }
    cudaError_t e = cudaMemsetAsync(workspace_device, 0, sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) return rs::cuda_fail(e, "status clear");
    return RS_OK;
}

int rs_set_status_mirror(int* host_word) {
    rs::DeviceInfo* di = nullptr;
    const int rc = rs::get_device(&di);
    if (rc) return rc;
    if ((uintptr_t)host_word & 3) return RS_ERR_POINTER;
    std::lock_guard<std::mutex> lk(rs::g_mu);
    di->mirror = host_word;
    return RS_OK;
}

int rs_set_dependent_launch(int on) {
    return (on == 0 || on == 1) ? rs::g_dependent_launch.exchange(on) : rs::g_dependent_launch.load();
}

uint32_t rs_set_wait_polls(uint32_t polls) {
    return polls ? rs::g_wait_polls.exchange(polls) : rs::g_wait_polls.load();
}

int rs_selftest_bounded_wait(void* workspace_device, uint32_t polls, void* stream) {
    if (!workspace_device || ((uintptr_t)workspace_device & 3)) return RS_ERR_POINTER;
    if (polls == 0 || polls > 4096) return RS_ERR_LIMIT;   // a self-test, not a delay loop
    rs::DeviceInfo* di = nullptr;
    const int rc = rs::get_device(&di);
    if (rc) return rc;
    rs::selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((int*)workspace_device, di->mirror, polls);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return rs::cuda_fail(e, "launch(selftest)");
    rs::g_launches.fetch_add(1, std::memory_order_relaxed);
    return RS_OK;
}

int rs_set_cluster_override(int cluster_ctas) {
    const bool valid = cluster_ctas == 0 || cluster_ctas == 1 || cluster_ctas == 2 || cluster_ctas == 4 ||
                       cluster_ctas == 8 || cluster_ctas == 16;
    return valid ? rs::g_cluster_override.exchange(cluster_ctas) : rs::g_cluster_override.load();
}

int rs_set_path_override(int mode) {
    return (mode >= 0 && mode <= 6) ? rs::g_path_override.exchange(mode) : rs::g_path_override.load();
}

uint64_t rs_kernel_launch_count(void) { return rs::g_launches.load(); }

const char* rs_status_string(int status) {
    switch (status) {
        case RS_OK: return "ok";
        case RS_ERR_DTYPE: return "Logits tensor must be of type float32 (FP32)";
        case RS_ERR_VOCAB: return "Vocabulary size must be multiple of 4, and no larger than 1048576";
        case RS_ERR_BATCH: return "B and T must be positive";
        case RS_ERR_TEMPERATURE: return "Temperature outside range, expect [0.001, 1000]";
        case RS_ERR_POINTER: return "null or misaligned pointer";
        case RS_ERR_WORKSPACE: return "workspace too small";
        case RS_ERR_CUDA: return "CUDA runtime error";
        case RS_ERR_TIMEOUT: return "a bounded on-chip wait gave up";
        case RS_ERR_LIMIT: return "size beyond what this entry point supports";
        case RS_ERR_INTERNAL: return "an invariant of the cutoff search was violated";
    }
    return "unknown status";
}

int rs_sample_static_scratch(const float* logits_device, int64_t B, int64_t T, int64_t V, float* penalties_device,
                             void* states_device, int32_t* out_device, double temperature, int64_t top_k, double top_p,
                             double presence_penalty, double repetition_penalty, double penalty_decay, void* stream) {
    return rs::sample_static_impl(logits_device, B, T, V, penalties_device, states_device, out_device, temperature, top_k,
                                  top_p, presence_penalty, repetition_penalty, penalty_decay, stream);
}

const char* rs_last_cuda_error(void) { return rs::g_err; }
const char* rs_version(void) { return "rapid_sampling_b200 0.1 (sm_100a)"; }

}  // extern "C"
