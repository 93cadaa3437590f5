// Row-per-CTA variant of the sampler for large batches (sm_100a).
//
// The reference runs one 1024-thread CTA per row (sampling.cu:500, :1025) and re-reads a global scratch copy of the
// row ~18 times.  Here a row is also handled by ONE CTA, so no value ever crosses an SM boundary, but:
//   * a thread plays LPT of the reference's 1024 "virtual lanes" (lane t still owns float4 groups t, t+1024, ... and
//     every fp32 sum keeps the reference's association: per-lane chain -> 32-lane xor tree -> warp values in order),
//     so a row costs 1024/LPT threads and several rows share an SM;
//   * every thread streams exactly the float4 groups it will read itself through a private pipeline of asynchronous
//     16-byte copies (cp.async) into shared memory: several stripes in flight per thread, no registers held by loads
//     in flight, and no barrier of any kind in the streaming passes.  The first stripes stay on chip as scaled logits,
//     so the second pass re-reads only the rest (from L2);
//   * the cutoff search runs on the short candidate list: first in one warp on exact integer masses, which settles
//     every row whose masses stay clear of top_p by more than the fp32 rounding of the reference's sums (nearly all);
//     else with the reference's fp32 sums, block-wide, one CTA barrier per evaluated round;
//   * with penalties, the first stripes of the update pass are already in flight while the search runs.
// Rows whose candidate list cannot settle the cutoff search the whole row on a global scratch row, dropping, in place
// and order-preserving, every element below the current lower bound as the bracket rises.
#include "rs_common.cuh"
#include "rs_rowcta.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>
#include <mutex>
#include <type_traits>

namespace rs {

namespace {

// shared-memory map (bytes)
constexpr int kOffScal = 0;        // s_idxt, s_token
constexpr int kOffCmd = 16;        // the search leader's command to the evaluating warps: 4 pivots, lo, hi, count at lo, go
constexpr int kOffFin = 48;        // the search's final state, published by the leader
constexpr int kOffWtot = 128;      // 32 warp totals of a scan
constexpr int kOffBoxC = 256;      // 2 x [16 physical warps][8 words]
constexpr int kOffBox = 1280;      // 2 x [4 values][32 virtual warps] floats, value-major
constexpr int kBoxBytes = 4 * 32 * 4;
constexpr int kOffQuick = kOffBox + 2 * kBoxBytes;   // the row's candidates as one unordered list of (bits of p, p in units of 2^-30)
static_assert(kOffQuick + kQuickCap * 8 <= kRowCtaFixedSmem, "fixed shared-memory area too small");
constexpr int kStripeBytes = 16384;   // 1024 float4 groups: one group per virtual lane

// order-preserving map float -> u32 (no NaN here: inputs are sanitised), so that integer warp reductions serve floats
__device__ __forceinline__ uint32_t fkey(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float fromkey(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// The xor trees (offsets 16, 8, 4, 2, 1) of N values per lane at once.  While more than one value is left, a lane
// keeps half of its partial sums and hands the other half to its partner -- the same additions as N separate
// butterflies, in N - 1 + log2(32 / N) shuffles -- so that m[0] ends as the total of value index (lane >> log2(32 / N)),
// identical in the lanes that share those bits.
template <int N, int O>
__device__ __forceinline__ void tree_levels(float* m, const int lane) {
    if constexpr (O > 0) {
        const bool up = (lane & O) != 0;
        if constexpr (N > 1) {
            constexpr int H = N / 2;
#pragma unroll
            for (int i = 0; i < H; i++) {
                const float keepv = up ? m[i + H] : m[i], give = up ? m[i] : m[i + H];
                m[i] = keepv + __shfl_xor_sync(0xffffffffu, give, O);
            }
            tree_levels<H, O / 2>(m, lane);
        } else {
            m[0] = m[0] + __shfl_xor_sync(0xffffffffu, m[0], O);
            tree_levels<1, O / 2>(m, lane);
        }
    }
}

}  // namespace

// LPT: virtual lanes per thread.  REP: the call has penalties (sampling.cu:172-438), else not (:517-964).  D: stages of
// a thread's copy pipeline.  NH: stages per stripe (2: a stage holds half a stripe, which buys twice the stages -- and
// bytes in flight -- from the same shared memory when two rows with penalties share an SM).  All compile-time, so that
// the streaming loops carry no tests on them.  LOWP: the logits are fp16 or bf16 (p.dtype says which); a group of four
// is then an 8-byte copy into the first half of the lane's 16-byte slot and is widened exactly to fp32 when it is read.
// Per-row parameters (p.rows) are a run-time matter: they only replace values that are kernel parameters anyway.
struct TagFull { static constexpr bool value = true; };
struct TagRagged { static constexpr bool value = false; };

template <int LPT, bool REP, int D, int NH, bool LOWP>
__global__ void __launch_bounds__(kLanes / LPT, (LPT >= 4 ? 2 : 1)) rowcta_kernel(const Params p, const RowCtaPlan pl) {
    constexpr int SL = LPT / NH;       // lanes of a thread that one copy stage serves (NH stages make up a stripe)
    constexpr int NT = kLanes / LPT;   // threads; thread t plays virtual lanes j * NT + t
    constexpr int WPB = NT / 32;       // warps; physical warp pw plays virtual warps j * WPB + pw
    constexpr int NV = LPT * 4;        // ordered masses a thread holds in a search round
    constexpr int CR = 2;              // candidates per virtual lane that are kept in registers during the search
    constexpr unsigned FULL = 0xffffffffu;
    extern __shared__ __align__(128) unsigned char smem[];
    const int t = threadIdx.x, lane = t & 31, pw = t >> 5;
    const int b = blockIdx.x;
    const int V = p.V, V4 = V >> 2;
    const int K = (V4 + kLanes - 1) >> 10;   // stripes of 1024 float4 groups
    // programmatic dependent launch: nothing in global memory is touched before the predecessor is complete and visible
    grid_dependents_may_launch();
    grid_dependency_wait();
    int a_kind = p.kind, a_top_k = p.top_k, a_sel_rank = p.sel_rank;
    float a_scale = p.scale, a_top_p = p.top_p;
    if (p.rows) {   // this row's own normalised parameters
        const RowArgs ra = p.rows[b];
        a_kind = ra.kind; a_top_k = ra.top_k; a_sel_rank = ra.sel_rank; a_scale = ra.scale; a_top_p = ra.top_p;
    }
    constexpr bool rep = REP;
    const bool use_cnt = (a_kind != kTopP);
    const char* lrow_b = reinterpret_cast<const char*>(p.logits) + (long long)b * p.row_stride * (LOWP ? 2 : 4);
    const float* lrow = reinterpret_cast<const float*>(lrow_b);      // as such for fp32 logits only
    const bool is_f16 = LOWP && p.dtype == RS_DTYPE_F16;
    // four logits of a group / one logit, widened exactly to fp32
    auto widen4 = [&](const uint2 r) -> float4 {
        if (is_f16) {
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
            const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
            return make_float4(a.x, a.y, c.x, c.y);
        }
        return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u), __uint_as_float(r.y << 16),
                           __uint_as_float(r.y & 0xffff0000u));
    };
    auto raw4 = [&](const unsigned char* slot16) -> float4 {        // a lane's 16-byte slot as it was copied
        if (!LOWP) return *reinterpret_cast<const float4*>(slot16);
        return widen4(*reinterpret_cast<const uint2*>(slot16));
    };
    auto logit1 = [&](int i) -> float {
        if (!LOWP) return lrow[i];
        const unsigned short h = reinterpret_cast<const unsigned short*>(lrow_b)[i];
        if (is_f16) return __half2float(__ushort_as_half(h));
        return __uint_as_float((uint32_t)h << 16);
    };
    float* prow = rep ? p.penalties + (long long)b * V : nullptr;
    const int NC = pl.cached, cap = pl.cap;

    int* s_idxt = reinterpret_cast<int*>(smem + kOffScal);
    int* s_token = reinterpret_cast<int*>(smem + kOffScal + 4);
    float* s_wtot = reinterpret_cast<float*>(smem + kOffWtot);
    float* cand = reinterpret_cast<float*>(smem + pl.off_cand);          // entry i of virtual lane v at cand[i * 1024 + v]
    unsigned char* ring = smem + pl.off_ring;                            // D stages of pl.stage_bytes
    unsigned char* cache = smem + pl.off_cache;                          // NC stripes of scaled logits
    uint32_t* s_ncl = reinterpret_cast<uint32_t*>(smem + kOffScal + 8);  // entries of the unordered candidate list
    uint2* qlist = reinterpret_cast<uint2*>(smem + kOffQuick);
    if (t == 0) {
        *s_idxt = 0;
        *s_token = 0;
        *s_ncl = 0u;
    }

    // ---- the thread's private copy pipeline ------------------------------------------------------------------
    // The n-th stripe requested in a pass lands in ring stage n % D (its logits in the first 16 KiB, its penalties in
    // the second), except that the logits of the first NC stripes go straight to their place in the on-chip cache.
    // A thread only ever copies, reads and overwrites its own 16-byte slots, so nothing but its own wait_group orders
    // anything.  Passes alternate their direction over the stripes (down, up, down): what one pass read last is what
    // the next one reads first, so a batch larger than L2 still finds the recent part of its rows there.
    const int Kf = V4 >> 10, rem = V4 & 1023;       // full stripes; float4 groups in the ragged last one (index Kf)
    bool tail_ok[LPT];
#pragma unroll
    for (int j = 0; j < LPT; j++) tail_ok[j] = (j * NT + t) < rem;
    constexpr uint32_t kPart = kStripeBytes / NH;              // bytes of logits (or of penalties) in a stage
    constexpr uint32_t kStage = REP ? 2 * kPart : kPart;
    const uint32_t sm_ring = smem_addr(ring) + (uint32_t)t * 16u, sm_cache = smem_addr(cache) + (uint32_t)t * 16u;
    const char* const gl = lrow_b + (size_t)t * (LOWP ? 8 : 16);   // this thread's group of stripe 0, lane j = 0
    const float4* const gp = reinterpret_cast<const float4*>(prow) + t;
    int ik = 0, ih = 0, islot = 0, idir = 1;   // next stripe (and part of it) to request, its stage, the direction of the pass
    // LG / PN: the pass wants the stripe's logits / penalties
    auto request = [&](auto lg_tag, auto pn_tag) {
        constexpr bool LG = decltype(lg_tag)::value, PN = decltype(pn_tag)::value;
        if ((unsigned)ik < (unsigned)K) {
            const uint32_t st = sm_ring + (uint32_t)islot * kStage;
            const bool keep = (ik < NC);
            const uint32_t ldst = keep ? sm_cache + (uint32_t)ik * kStripeBytes : st;
            const char* src = gl + (size_t)ik * kLanes * (LOWP ? 8 : 16);
            const float4* psrc = gp + (size_t)ik * kLanes;
            const bool fullk = ik < Kf;
#pragma unroll
            for (int h = 0; h < NH; h++) {
                if (NH == 1 || h == ih) {
#pragma unroll
                    for (int jj = 0; jj < SL; jj++) {
                        const int j = h * SL + jj;
                        if (fullk || tail_ok[j]) {
                            // a kept stripe has the stripe's own layout, a stage holds only this part's lanes
                            if (LG) {
                                if (LOWP) cp_async8(ldst + (keep ? j : jj) * NT * 16, src + (size_t)j * NT * 8);
                                else cp_async16(ldst + (keep ? j : jj) * NT * 16, src + (size_t)j * NT * 16);
                            }
                            if (PN) cp_async16(st + kPart + jj * NT * 16, psrc + j * NT);
                        }
                    }
                }
            }
        }
        cp_commit();
        if (NH == 1 || ++ih == NH) {
            ih = 0;
            ik += idir;
        }
        islot = (islot + 1 == D) ? 0 : islot + 1;
    };
    auto wait_stage = [&]() {   // the oldest requested stage has landed
        asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory");
    };
    auto begin_pass = [&](const int first, const int dir, auto lg_tag, auto pn_tag) {
        ik = first;
        ih = 0;
        idir = dir;
        islot = 0;
#pragma unroll
        for (int i = 0; i < D - 1; i++) request(lg_tag, pn_tag);
    };
    using Yes = TagFull;
    using No = TagRagged;
    using Pen = std::conditional_t<REP, TagFull, TagRagged>;
    begin_pass(K - 1, -1, Yes(), Pen());

    // exchange of warp values inside the CTA: two alternating boxes, one barrier per exchange
    int phase = 0;
    auto box_of = [&](int ph) -> float* { return reinterpret_cast<float*>(smem + kOffBox + ph * kBoxBytes); };
    auto boxc_of = [&](int ph) -> uint32_t* { return reinterpret_cast<uint32_t*>(smem + kOffBoxC + ph * 16 * 8 * 4); };

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

    RngWords rng;
    {
        const uint4* st = reinterpret_cast<const uint4*>(p.states + (long long)b * RS_STATE_BYTES);
        rng.ctr = st[0]; rng.block = st[1]; rng.key_pos = st[2];
    }
    uint32_t rnd4[4], r0, r1;
    rng_peek2(rng, r0, r1, rnd4);
    const float ux = u01(r0), uy = u01(r1);

    // x of one float4 group as the streaming passes compute it, read from global memory (slow paths only)
    auto xload_global = [&](int g) -> float4 {
        float4 v = LOWP ? widen4(__ldg(reinterpret_cast<const uint2*>(lrow_b) + g)) : __ldg(reinterpret_cast<const float4*>(lrow) + g);
        if (rep) v = scaled4_rep(v, __ldcg(reinterpret_cast<const float4*>(prow) + g), a_scale);
        else v = scaled4(v, a_scale);
        return v;
    };

    // ---- pass 1: x = sanitised scaled logit (sampling.cu:208-227, :547-559); every virtual lane's maximum ----
    float tmax[LPT];
#pragma unroll
    for (int j = 0; j < LPT; j++) tmax[j] = -INFINITY;
    {
        int cslot = 0;
        auto stripe = [&](auto full_tag, const int k) {
            constexpr bool FULLK = decltype(full_tag)::value;
            const bool keep = (k < NC);
            unsigned char* own = cache + (size_t)k * kStripeBytes;
#pragma unroll
            for (int h = 0; h < NH; h++) {
                request(Yes(), Pen());
                wait_stage();
                const unsigned char* st = ring + (size_t)cslot * kStage;
                if (FULLK) {   // the groups of a stage together, with one test for Inf / NaN products (see stream_x)
                    float4 l[SL], q[SL], v[SL];
                    float probe = 0.f;
#pragma unroll
                    for (int jj = 0; jj < SL; jj++) {
                        const int j = h * SL + jj;
                        l[jj] = keep ? raw4(own + (size_t)(j * NT + t) * 16) : raw4(st + (size_t)(jj * NT + t) * 16);
                        if (REP) {
                            q[jj] = reinterpret_cast<const float4*>(st + kPart)[jj * NT + t];
                            v[jj] = make_float4((l[jj].x - q[jj].x) * a_scale, (l[jj].y - q[jj].y) * a_scale, (l[jj].z - q[jj].z) * a_scale,
                                                (l[jj].w - q[jj].w) * a_scale);
                        } else {
                            v[jj] = make_float4(l[jj].x * a_scale, l[jj].y * a_scale, l[jj].z * a_scale, l[jj].w * a_scale);
                        }
                        probe += fmaf(v[jj].w, 0.f, fmaf(v[jj].z, 0.f, fmaf(v[jj].y, 0.f, v[jj].x * 0.f)));
                    }
                    if (probe != probe) {
#pragma unroll
                        for (int jj = 0; jj < SL; jj++) v[jj] = REP ? scaled4_rep(l[jj], q[jj], a_scale) : scaled4(l[jj], a_scale);
                    }
#pragma unroll
                    for (int jj = 0; jj < SL; jj++) {
                        const int j = h * SL + jj;
                        tmax[j] = fmaxf(fmaxf(fmaxf(tmax[j], v[jj].x), fmaxf(v[jj].y, v[jj].z)), v[jj].w);
                        if (keep) reinterpret_cast<float4*>(own)[j * NT + t] = v[jj];
                    }
                } else {
#pragma unroll
                    for (int jj = 0; jj < SL; jj++) {
                        const int j = h * SL + jj;
                        if (tail_ok[j]) {
                            float4 v = keep ? raw4(own + (size_t)(j * NT + t) * 16) : raw4(st + (size_t)(jj * NT + t) * 16);
                            if (REP) v = scaled4_rep(v, reinterpret_cast<const float4*>(st + kPart)[jj * NT + t], a_scale);
                            else v = scaled4(v, a_scale);
                            tmax[j] = fmaxf(fmaxf(fmaxf(tmax[j], v.x), fmaxf(v.y, v.z)), v.w);
                            if (keep) reinterpret_cast<float4*>(own)[j * NT + t] = v;
                        }
                    }
                }
                cslot = (cslot + 1 == D) ? 0 : cslot + 1;
            }
        };
        if (rem) stripe(TagRagged(), Kf);
        for (int k = Kf - 1; k >= 0; k--) stripe(TagFull(), k);
    }
    begin_pass(NC, 1, Yes(), Pen());   // the second pass's first stripes travel while the maxima are reduced
    stamp(1);
    stamp(2);
    // row maximum, and per virtual warp its sel_rank-th largest lane maximum: at least sel_rank elements of that
    // warp are >= it, so the minimum over the warps bounds 32 * sel_rank elements of the row from below
    const int sel_rank = a_sel_rank;
    float mx, beta_x;
    {
        uint32_t* box = reinterpret_cast<uint32_t*>(box_of(phase));
#pragma unroll
        for (int j = 0; j < LPT; j++) {
            const uint32_t key = fkey(tmax[j]);
            uint32_t top = __reduce_max_sync(FULL, key), sel = top, cur = key;
            for (int r = 1; r < sel_rank; r++) {     // drop one occurrence of the current maximum, take the next
                const unsigned m = __ballot_sync(FULL, cur == sel);
                if (lane == __ffs(m) - 1) cur = 0u;
                sel = __reduce_max_sync(FULL, cur);
            }
            if (lane == 0) {
                box[j * WPB + pw] = top;
                box[32 + j * WPB + pw] = sel;
            }
        }
        __syncthreads();
        mx = fromkey(__reduce_max_sync(FULL, box[lane]));
        beta_x = fromkey(__reduce_min_sync(FULL, box[32 + lane]));
        phase ^= 1;
    }
    stamp(3);
    const bool try_cand = (sel_rank > 0);
    float beta_e = try_cand ? exp2f(beta_x - mx) : INFINITY;

    // ---- pass 2: e = exp2f(x - max), ordered denominator (sampling.cu:560-572); min / max of e; elements with
    // e >= beta_e are appended, in order, to their lane's candidate list.  A list that looks too thin to settle the
    // cutoff gets its bound lowered 16-fold and the pass repeated (from global memory), at most twice. ------------
    float acc[LPT], emin, emax, csum, denom;
    int nc[LPT], ns;
    bool cand_ok;
    uint32_t ncand, nstrict;
    auto pass2_group = [&](const int j, float4 v) {
        v.x = exp2f(v.x - mx);
        v.y = exp2f(v.y - mx);
        v.z = exp2f(v.z - mx);
        v.w = exp2f(v.w - mx);
        float em = 0.f;
        em += v.x; em += v.y; em += v.z; em += v.w;
        acc[j] += em;
        const float hi = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
        emin = fminf(fminf(emin, fminf(v.x, v.y)), fminf(v.z, v.w));
        emax = fmaxf(emax, hi);
        if (hi >= beta_e) {
            const float e4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                if (e4[q] >= beta_e) {
                    if (nc[j] < cap) cand[nc[j] * kLanes + j * NT + t] = e4[q];
                    nc[j]++;
                    ns += (e4[q] > beta_e) ? 1 : 0;
                }
            }
            csum += (v.x >= beta_e ? v.x : 0.f) + (v.y >= beta_e ? v.y : 0.f) + (v.z >= beta_e ? v.z : 0.f) +
                    (v.w >= beta_e ? v.w : 0.f);
        }
    };
    // One pass over the row as scaled logits x, stripes in ascending order (every lane's chain order): the kept
    // stripes from shared memory, the rest through the copy pipeline (which begin_pass(NC, 1, ...) has started).
    // fn(j, k, v) gets one group; the groups of a full stripe's stage go to fn_batch(h, k, v[SL]) together, scaled with
    // ONE test for Inf / NaN products per stage (x * 0 is NaN exactly for those): a branch per group would end the
    // basic block there, and the few warps of a row would wait out every dependent instruction of every group.
    auto stream_x = [&](auto&& fn, auto&& fn_batch) {
        int cslot = 0;
        auto stripe = [&](auto full_tag, const int k) {
            constexpr bool FULLK = decltype(full_tag)::value;
            const bool kept = (k < NC);
            const unsigned char* own = cache + (size_t)k * kStripeBytes;
#pragma unroll
            for (int h = 0; h < NH; h++) {
                const unsigned char* st = ring + (size_t)cslot * kStage;
                if (!kept) {
                    request(Yes(), Pen());
                    wait_stage();
                    cslot = (cslot + 1 == D) ? 0 : cslot + 1;
                }
                if (FULLK) {
                    float4 v[SL];
                    if (kept) {
#pragma unroll
                        for (int jj = 0; jj < SL; jj++) v[jj] = reinterpret_cast<const float4*>(own)[(h * SL + jj) * NT + t];
                    } else {
                        float4 l[SL], q[SL];
                        float probe = 0.f;
#pragma unroll
                        for (int jj = 0; jj < SL; jj++) {
                            l[jj] = raw4(st + (size_t)(jj * NT + t) * 16);
                            if (REP) {
                                q[jj] = reinterpret_cast<const float4*>(st + kPart)[jj * NT + t];
                                v[jj] = make_float4((l[jj].x - q[jj].x) * a_scale, (l[jj].y - q[jj].y) * a_scale, (l[jj].z - q[jj].z) * a_scale,
                                                    (l[jj].w - q[jj].w) * a_scale);
                            } else {
                                v[jj] = make_float4(l[jj].x * a_scale, l[jj].y * a_scale, l[jj].z * a_scale, l[jj].w * a_scale);
                            }
                            probe += fmaf(v[jj].w, 0.f, fmaf(v[jj].z, 0.f, fmaf(v[jj].y, 0.f, v[jj].x * 0.f)));
                        }
                        if (probe != probe) {   // rare: the exact formulas, group by group
#pragma unroll
                            for (int jj = 0; jj < SL; jj++) v[jj] = REP ? scaled4_rep(l[jj], q[jj], a_scale) : scaled4(l[jj], a_scale);
                        }
                    }
                    fn_batch(h, k, v);
                } else {
#pragma unroll
                    for (int jj = 0; jj < SL; jj++) {
                        const int j = h * SL + jj;
                        if (tail_ok[j]) {
                            float4 v = kept ? reinterpret_cast<const float4*>(own)[j * NT + t] : raw4(st + (size_t)(jj * NT + t) * 16);
                            if (!kept) {
                                if (REP) v = scaled4_rep(v, reinterpret_cast<const float4*>(st + kPart)[jj * NT + t], a_scale);
                                else v = scaled4(v, a_scale);
                            }
                            fn(j, k, v);
                        }
                    }
                }
            }
        };
        for (int k = 0; k < Kf; k++) stripe(TagFull(), k);
        if (rem) stripe(TagRagged(), Kf);
    };
    auto pass2 = [&](const bool last) -> bool {
        emin = INFINITY; emax = -INFINITY; csum = 0.f; ns = 0;
#pragma unroll
        for (int j = 0; j < LPT; j++) { acc[j] = 0.f; nc[j] = 0; }
        stream_x([&](const int j, const int, const float4 v) { pass2_group(j, v); },
                 [&](const int h, const int, float4 (&v)[SL]) {
                     // the groups of one stage: every lane's sum in its own order, one test for candidates
                     float hi[SL], hi_all = 0.f;
#pragma unroll
                     for (int jj = 0; jj < SL; jj++) {
                         const int j = h * SL + jj;
                         v[jj].x = exp2f(v[jj].x - mx);
                         v[jj].y = exp2f(v[jj].y - mx);
                         v[jj].z = exp2f(v[jj].z - mx);
                         v[jj].w = exp2f(v[jj].w - mx);
                         float em = 0.f;
                         em += v[jj].x; em += v[jj].y; em += v[jj].z; em += v[jj].w;
                         acc[j] += em;
                         hi[jj] = fmaxf(fmaxf(v[jj].x, v[jj].y), fmaxf(v[jj].z, v[jj].w));
                         emin = fminf(fminf(emin, fminf(v[jj].x, v[jj].y)), fminf(v[jj].z, v[jj].w));
                         emax = fmaxf(emax, hi[jj]);
                         hi_all = fmaxf(hi_all, hi[jj]);
                     }
                     if (hi_all >= beta_e) {
#pragma unroll
                         for (int jj = 0; jj < SL; jj++) {
                             const int j = h * SL + jj;
                             if (hi[jj] >= beta_e) {
                                 const float e4[4] = {v[jj].x, v[jj].y, v[jj].z, v[jj].w};
#pragma unroll
                                 for (int q = 0; q < 4; q++) {
                                     if (e4[q] >= beta_e) {
                                         if (nc[j] < cap) cand[nc[j] * kLanes + j * NT + t] = e4[q];
                                         nc[j]++;
                                         ns += (e4[q] > beta_e) ? 1 : 0;
                                     }
                                 }
                                 csum += (v[jj].x >= beta_e ? v[jj].x : 0.f) + (v[jj].y >= beta_e ? v[jj].y : 0.f) +
                                         (v[jj].z >= beta_e ? v[jj].z : 0.f) + (v[jj].w >= beta_e ? v[jj].w : 0.f);
                             }
                         }
                     }
                 });
        stamp(4);
        float* box = box_of(phase);
        uint32_t* boxc = boxc_of(phase);
        int nct = 0;
        bool over = false;
#pragma unroll
        for (int j = 0; j < LPT; j++) {
            const float a = warp_tree_sum(acc[j]);
            if (lane == 0) box[j * WPB + pw] = a;
            nct += nc[j];
            over = over || (nc[j] > cap);
        }
        const uint32_t kmin = __reduce_min_sync(FULL, fkey(emin)), kmax = __reduce_max_sync(FULL, fkey(emax));
        const uint32_t wov = __any_sync(FULL, over) ? 1u : 0u;
        const uint32_t wnc = __reduce_add_sync(FULL, (uint32_t)nct), wns = __reduce_add_sync(FULL, (uint32_t)ns);
        const float wcs = warp_tree_sum(csum);
        if (lane == 0) {
            boxc[pw * 8 + 0] = kmin; boxc[pw * 8 + 1] = kmax; boxc[pw * 8 + 2] = wov;
            boxc[pw * 8 + 3] = wnc; boxc[pw * 8 + 4] = wns; boxc[pw * 8 + 5] = __float_as_uint(wcs);
        }
        __syncthreads();
        denom = warp_tree_sum(box[lane]);   // tree over the 32 warp partials (sampling.cu:29-33)
        const bool in = lane < WPB;
        emin = fromkey(__reduce_min_sync(FULL, in ? boxc[lane * 8 + 0] : 0xffffffffu));
        emax = fromkey(__reduce_max_sync(FULL, in ? boxc[lane * 8 + 1] : 0u));
        cand_ok = try_cand && (__reduce_add_sync(FULL, in ? boxc[lane * 8 + 2] : 0u) == 0u);
        ncand = __reduce_add_sync(FULL, in ? boxc[lane * 8 + 3] : 0u);
        nstrict = __reduce_add_sync(FULL, in ? boxc[lane * 8 + 4] : 0u);
        const float cmass = warp_tree_sum(in ? __uint_as_float(boxc[lane * 8 + 5]) : 0.f) / denom;   // a forecast only
        phase ^= 1;
        const bool enough = (use_cnt && nstrict > (uint32_t)a_top_k) || cmass > a_top_p * 1.001f;
        return !cand_ok || enough || last || !(beta_e > 0.f);
    };
    for (int attempt = 0; attempt < 3; attempt++) {
        if (pass2(attempt == 2)) break;
        if (attempt == 0) {
            const bool all_in = beta_e * 0.0625f <= emin;      // a flat row: the lowered bound would admit every element
            if (all_in && V > cap * kLanes) {
                cand_ok = false;
                break;
            }
            beta_e = all_in ? 0.f : beta_e * 0.0625f;
        } else {
            beta_e *= 0.0625f;
        }
        begin_pass(NC, 1, Yes(), Pen());   // the same pass again with the lowered bound
    }
    if (REP) begin_pass(K - 1, -1, No(), Yes());   // the update pass's first penalty stripes, in flight from here on
    const float pmin = emin / denom, pmax = emax / denom;   // division is monotone
    if (p.dbg_probs) {   // test instrumentation: the probabilities of the whole row
        float* dprow = p.dbg_probs + (long long)b * V;
        for (int k = 0; k < K; k++)
#pragma unroll
            for (int j = 0; j < LPT; j++) {
                const int g = k * kLanes + j * NT + t;
                if (g < V4) {
                    float4 v = xload_global(g);
                    v.x = exp2f(v.x - mx) / denom; v.y = exp2f(v.y - mx) / denom;
                    v.z = exp2f(v.z - mx) / denom; v.w = exp2f(v.w - mx) / denom;
                    reinterpret_cast<float4*>(dprow)[g] = v;
                }
            }
    }
    stamp(5);

    // ---- row totals of NV ordered masses (4 pivots x LPT lanes per thread), 4 counts and min / max of two bit
    // patterns.  Masses: xor tree over the 32 lanes of each virtual warp -- all trees share shuffles -- then the 32
    // warp values added in warp order, as thread 0 of the reference does (sampling.cu:34-42): lanes 0..3 of every
    // warp run the four 32-step chains on vector loads, lanes 4..9 add up the counts and bounds, and the ten results
    // reach the other lanes by shuffles.
    auto publish_partials = [&](float (&m)[NV], const uint32_t (&c)[4], uint32_t mn, uint32_t mxv) {
        tree_levels<NV, 16>(m, lane);
        // value index i = j * 4 + pivot ended in the lanes whose upper bits spell i
        constexpr int SH = (NV == 32) ? 0 : (NV == 16) ? 1 : (NV == 8) ? 2 : 3;
        uint32_t cs[4];
#pragma unroll
        for (int i = 0; i < 4; i++) cs[i] = __reduce_add_sync(FULL, c[i]);
        mn = __reduce_min_sync(FULL, mn);
        mxv = __reduce_max_sync(FULL, mxv);
        float* box = box_of(phase);
        uint32_t* boxc = boxc_of(phase);
        if ((lane & ((1 << SH) - 1)) == 0) {
            const int i = lane >> SH;
            box[(i & 3) * 32 + (i >> 2) * WPB + pw] = m[0];
        }
        if (lane == 0) {
            *reinterpret_cast<uint4*>(boxc + pw * 8) = make_uint4(cs[0], cs[1], cs[2], cs[3]);
            *reinterpret_cast<uint2*>(boxc + pw * 8 + 4) = make_uint2(mn, mxv);
        }
    };
    auto combine_partials = [&](uint32_t (&cnt)[4], float (&mass)[4], uint32_t& vmin, uint32_t& vmax) {
        const float* box = box_of(phase);
        const uint32_t* boxc = boxc_of(phase);
        uint32_t r = 0u;
        if (lane < 4) {
            const float4* col = reinterpret_cast<const float4*>(box + lane * 32);
            float4 w[8];
#pragma unroll
            for (int q = 0; q < 8; q++) w[q] = col[q];
            float sacc = w[0].x;
            sacc += w[0].y; sacc += w[0].z; sacc += w[0].w;
#pragma unroll
            for (int q = 1; q < 8; q++) { sacc += w[q].x; sacc += w[q].y; sacc += w[q].z; sacc += w[q].w; }
            r = __float_as_uint(sacc);
        } else if (lane < 10) {
            const int f = lane - 4;
            uint32_t a = boxc[f];
#pragma unroll
            for (int w = 1; w < WPB; w++) {
                const uint32_t x = boxc[w * 8 + f];
                a = (f < 4) ? a + x : (f == 4) ? min(a, x) : max(a, x);
            }
            r = a;
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            mass[i] = __uint_as_float(__shfl_sync(FULL, r, i));
            cnt[i] = __shfl_sync(FULL, r, 4 + i);
        }
        vmin = __shfl_sync(FULL, r, 8);
        vmax = __shfl_sync(FULL, r, 9);
    };
    auto totals = [&](float (&m)[NV], const uint32_t (&c)[4], uint32_t mn, uint32_t mxv, uint32_t (&cnt)[4], float (&mass)[4],
                      uint32_t& vmin, uint32_t& vmax) {
        publish_partials(m, c, mn, mxv);
        __syncthreads();
        combine_partials(cnt, mass, vmin, vmax);
        phase ^= 1;
    };

    // ---- cutoff search (sampling.cu:593-654, :829-878): the reference's loop replayed with the same pivots and the
    // same decisions; see the cluster variant for why the candidate list answers every pivot the same way -----------
    const uint32_t top_k = (uint32_t)a_top_k;
    const float top_p = a_top_p;
    uint32_t left = 0, right = 0, rounds = 0, n_eval = 0;
    uint32_t path = 1;
    uint32_t conv_cnt = 0, conv_left_cnt = 0;
    float conv_mass = 0.f;
    // Warp 0 leads: it alone replays the reference's loop -- pivots, tests, bracket updates, the rounds that need no
    // data -- and, when a round needs sums, publishes its four pivots; every warp then evaluates its own lanes, reduces
    // them and stores the warp values, and only the leader adds them up.  Two named barriers per evaluated round:
    // "partials stored" (the others only arrive) and "next command published".
    //  * clamp (candidate list only): every probability above beta_p is on the list, so a pivot above beta_p sees exactly
    //    the elements the reference sees.  A pivot u <= beta_p is not evaluated; instead the set {p > beta_p} is: if it
    //    already holds more than top_k elements or more than top_p mass, so does the larger set {p >= u}, the reference's
    //    test at u fails and its carried state keeps the loop going -- all it uses these values for.  Otherwise: not valid.
    //  * frozen (candidate list only): once every element strictly inside (left, right) has one and the same value v, the
    //    remaining rounds need no data: a pivot equal to `left` selects the set of `left`, a pivot in (left, v] the set
    //    {p >= v}, a pivot above v the set of `right`.
    volatile uint32_t* s_cmd = reinterpret_cast<volatile uint32_t*>(smem + kOffCmd);
    volatile uint32_t* s_fin = reinterpret_cast<volatile uint32_t*>(smem + kOffFin);
    auto run_search = [&](auto&& lane_eval, const bool clamp, const uint32_t beta_p, const bool sure_cnt,
                          const uint32_t n_above) -> bool {
        const uint32_t ustar = clamp ? beta_p + 1u : 0u;
        // leader state
        uint32_t l_left = __float_as_uint(pmin), l_right = __float_as_uint(pmax) + 1u, l_rounds = 0, l_evals = 0;
        uint32_t cnt_x = (uint32_t)V, cnt_r = 0u;
        float mass_x = 1.0f, mass_r = 0.f;
        bool frozen = false, valid = true, have_vals = false, waiting = false;
        uint32_t v_bits = 0, cnt_v = 0;
        float mass_v = 0.f;
        uint32_t pv[3] = {0u, 0u, 0u};
        uint32_t cnt[4] = {0u, 0u, 0u, 0u};
        float mass[4] = {0.f, 0.f, 0.f, 0.f};
        for (;;) {
            if (pw == 0) {
                bool finished = false;
                if (waiting) {    // the sums of the round that was asked for
                    uint32_t vmin, vmax;
                    combine_partials(cnt, mass, vmin, vmax);
                    if (clamp && l_left >= beta_p && vmin >= vmax) {   // one distinct value inside (none: vmin > vmax)
                        frozen = true;
                        v_bits = (vmin == vmax) ? vmin : l_left;
                        cnt_v = cnt[3];      // the set {p >= left + 1} is {p >= v}
                        mass_v = mass[3];
                    }
                    have_vals = true;
                    waiting = false;
                }
                for (;;) {
                    if (have_vals) {   // the three tests and the bracket update (sampling.cu:618-651)
                        have_vals = false;
                        bool ok[3], bad = false;
#pragma unroll
                        for (int i = 0; i < 3; i++) {
                            const bool below = clamp && pv[i] <= beta_p;
                            const bool exceeds = (use_cnt && cnt[i] > top_k) || mass[i] > top_p;
                            const bool pass = (!use_cnt || cnt[i] < top_k) && mass[i] < top_p;
                            ok[i] = !below && pass;
                            bad = bad || (below && !exceeds);
                        }
                        if (bad) { valid = false; finished = true; break; }
                        const bool s0 = ok[0], s1 = !s0 && ok[1], s2 = !s0 && !s1 && ok[2];
                        const uint32_t nl = s0 ? l_left : s1 ? pv[0] : s2 ? pv[1] : pv[2];
                        const uint32_t nr = s0 ? pv[0] : s1 ? pv[1] : s2 ? pv[2] : l_right;
                        const uint32_t ncx = s0 ? cnt_x : s1 ? cnt[0] : s2 ? cnt[1] : cnt[2];
                        const float nmx = s0 ? mass_x : s1 ? mass[0] : s2 ? mass[1] : mass[2];
                        const uint32_t ncr = s0 ? cnt[0] : s1 ? cnt[1] : s2 ? cnt[2] : cnt_r;
                        const float nmr = s0 ? mass[0] : s1 ? mass[1] : s2 ? mass[2] : mass_r;
                        l_left = nl; l_right = nr; cnt_x = ncx; mass_x = nmx; cnt_r = ncr; mass_r = nmr;
                    }
                    const bool go = use_cnt ? (cnt_x > top_k || mass_x > top_p) : (mass_x > top_p);
                    if (!(go && l_left < l_right - 1u) || l_rounds >= 64u) { finished = true; break; }
                    l_rounds++;
                    const uint32_t pz = (l_left + l_right) >> 1, py = (l_left + pz) >> 1, pwv = (pz + l_right) >> 1;
                    pv[0] = py; pv[1] = pz; pv[2] = pwv;
                    if (clamp && sure_cnt && pwv <= beta_p) {
                        // all three pivots lie at or below the bound, and more than top_k elements are known to lie
                        // strictly above it: every test fails, the lower end moves to the last pivot, no data is needed
                        l_left = pwv;
                        cnt_x = n_above;
                        mass_x = 0.f;
                        continue;
                    }
                    if (frozen) {
#pragma unroll
                        for (int i = 0; i < 3; i++) {
                            const bool at_left = (pv[i] == l_left), le_v = (pv[i] <= v_bits);
                            cnt[i] = at_left ? cnt_x : le_v ? cnt_v : cnt_r;
                            mass[i] = at_left ? mass_x : le_v ? mass_v : mass_r;
                        }
                        have_vals = true;
                        continue;
                    }
                    l_evals++;
                    waiting = true;
                    break;
                }
                if (lane == 0) {
                    if (waiting) {
                        s_cmd[0] = max(pv[0], ustar); s_cmd[1] = max(pv[1], ustar); s_cmd[2] = max(pv[2], ustar);
                        s_cmd[3] = max(l_left + 1u, ustar);
                        s_cmd[4] = l_left; s_cmd[5] = l_right; s_cmd[6] = cnt_x; s_cmd[7] = 1u;
                    } else {
                        s_cmd[7] = 0u;
                        s_fin[0] = l_left; s_fin[1] = l_right; s_fin[2] = l_rounds; s_fin[3] = l_evals;
                        s_fin[4] = cnt_r; s_fin[5] = cnt_x; s_fin[6] = __float_as_uint(mass_r); s_fin[7] = valid ? 1u : 0u;
                    }
                }
                (void)finished;
            }
            asm volatile("bar.sync 2, %0;" ::"n"(NT) : "memory");      // command published
            if (s_cmd[7] == 0u) break;
            {
                const float f[4] = {__uint_as_float(s_cmd[0]), __uint_as_float(s_cmd[1]), __uint_as_float(s_cmd[2]),
                                    __uint_as_float(s_cmd[3])};
                const uint32_t lo = s_cmd[4], hi = s_cmd[5], cnt_lo = s_cmd[6];
                float m[NV];
                uint32_t c[4], mn, mxv;
                lane_eval(f, lo, hi, cnt_lo, m, c, mn, mxv);
                publish_partials(m, c, mn, mxv);
            }
            if (pw == 0) asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory");      // partials stored: the leader waits,
            else asm volatile("bar.arrive 1, %0;" ::"n"(NT) : "memory");            // the others go on to the next command
        }
        left = s_fin[0]; right = s_fin[1]; rounds = s_fin[2]; n_eval += s_fin[3];
        conv_cnt = s_fin[4];
        conv_left_cnt = s_fin[5];
        conv_mass = __uint_as_float(s_fin[6]);
        const bool was_valid = s_fin[7] != 0u;
        __syncthreads();     // everybody has read the final state before anything reuses the exchange area
        return was_valid && (!clamp || left > beta_p);
    };

    float gtp[LPT];          // per virtual lane: mass above the threshold, ties with it, count above
    uint32_t eqk[LPT], gtk[LPT];
#pragma unroll
    for (int j = 0; j < LPT; j++) { gtp[j] = 0.f; eqk[j] = 0u; gtk[j] = 0u; }
    // Two attempts share one copy of the search loop: the candidate lists first (the first CR probabilities of every
    // lane's list live in registers for the rounds -- unused places hold -1, which no pivot admits -- longer lists
    // continue in shared memory), then, if they cannot settle the cutoff, the whole row on the global scratch row.
    int m_own[LPT], n_row[LPT];
    float creg[LPT][CR];
    Row<1, false> row;
    row.slab = reinterpret_cast<float4*>(p.scratch + (long long)b * V);
    row.t = t;
    row.tg = t;
    bool long_lists = false;
    uint32_t beta_p = 0u;
    uint32_t list_total = (uint32_t)V, list_left = 0u;
    bool whole = false;
    int quick = 0;           // outcome of the one-warp search on integer masses: 0 not settled that way, 1 settled, 2 list too short
    auto lane_eval = [&](const float (&f)[4], uint32_t lo, uint32_t hi, uint32_t cnt_lo, float (&m)[NV], uint32_t (&c)[4],
                         uint32_t& mn, uint32_t& mxv) {
        c[0] = c[1] = c[2] = c[3] = 0u;
        if (!whole) {
            mn = 0xffffffffu;
            mxv = 0u;
#pragma unroll
            for (int j = 0; j < LPT; j++) {
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int i = 0; i < CR; i++) {
                    const float q = creg[j][i];
                    const uint32_t qb = __float_as_uint(q);
                    if (q >= f[0]) { c[0]++; a0 += q; }
                    if (q >= f[1]) { c[1]++; a1 += q; }
                    if (q >= f[2]) { c[2]++; a2 += q; }
                    if (q >= f[3]) { c[3]++; a3 += q; }
                    if (qb > lo && qb < hi) { mn = min(mn, qb); mxv = max(mxv, qb); }
                }
                if (long_lists) {
                    for (int i = CR; i < m_own[j]; i++) {
                        const float q = cand[i * kLanes + j * NT + t];
                        const uint32_t qb = __float_as_uint(q);
                        if (q >= f[0]) { c[0]++; a0 += q; }
                        if (q >= f[1]) { c[1]++; a1 += q; }
                        if (q >= f[2]) { c[2]++; a2 += q; }
                        if (q >= f[3]) { c[3]++; a3 += q; }
                        if (qb > lo && qb < hi) { mn = min(mn, qb); mxv = max(mxv, qb); }
                    }
                }
                m[j * 4 + 0] = a0; m[j * 4 + 1] = a1; m[j * 4 + 2] = a2; m[j * 4 + 3] = a3;
            }
        } else {
            mn = 0u;
            mxv = 1u;   // bounds are not tracked on the whole row
            const bool compact = (lo != list_left) && (cnt_lo * 2u <= list_total);
#pragma unroll
            for (int j = 0; j < LPT; j++) {
                float mj[4];
                uint32_t c01, c23;
                row.tg = j * NT + t;
                if (compact) slab_pass<1, false, true>(row, n_row[j], f, __uint_as_float(lo), mj, c01, c23);
                else slab_pass<1, false, false>(row, n_row[j], f, 0.f, mj, c01, c23);
                m[j * 4 + 0] = mj[0]; m[j * 4 + 1] = mj[1]; m[j * 4 + 2] = mj[2]; m[j * 4 + 3] = 0.f;
                c[0] += c01 & 0xffffu; c[1] += c01 >> 16; c[2] += c23 & 0xffffu;
            }
            if (compact) { list_total = cnt_lo; list_left = lo; }
        }
    };
    for (int attempt = cand_ok ? 0 : 1; attempt < 2; attempt++) {
        whole = (attempt == 1);
        if (!whole) {
            int m_max = 0, mine = 0;
#pragma unroll
            for (int j = 0; j < LPT; j++) {
                m_own[j] = min(nc[j], cap);
                m_max = max(m_max, m_own[j]);
                mine += m_own[j];
            }
            // a place for this thread's entries in the row's unordered list (short lists only)
            const bool listed = p.quick && ncand <= (uint32_t)kQuickCap;
            uint32_t at = 0u;
            if (listed) {
                uint32_t incl = (uint32_t)mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t v = __shfl_up_sync(FULL, incl, o);
                    if (lane >= o) incl += v;
                }
                uint32_t base = 0u;
                if (lane == 31 && incl) base = atomicAdd(s_ncl, incl);
                at = __shfl_sync(FULL, base, 31) + incl - (uint32_t)mine;
            }
#pragma unroll
            for (int j = 0; j < LPT; j++) {
#pragma unroll
                for (int i = 0; i < CR; i++) creg[j][i] = -1.f;
                for (int i = 0; i < m_own[j]; i++) {
                    const float q = cand[i * kLanes + j * NT + t] / denom;
                    cand[i * kLanes + j * NT + t] = q;
                    if (listed) qlist[at++] = make_uint2(__float_as_uint(q), __float2uint_rn(q * 1073741824.f));
#pragma unroll
                    for (int r = 0; r < CR; r++)
                        if (i == r) creg[j][r] = q;
                }
            }
            long_lists = __any_sync(FULL, m_max > CR);
            beta_p = __float_as_uint(beta_e / denom);
            if (listed) {
                // ---- first try: the whole search in warp 0, on integer masses (quick_search)
                __syncthreads();
                if (pw == 0) {
                    uint32_t ql, qr, qn;
                    const int verdict = quick_search<false>(qlist, min(*s_ncl, (uint32_t)kQuickCap), lane, cap + 38, use_cnt, top_k, top_p, beta_p,
                                                     pmin, pmax, (uint32_t)V, ql, qr, qn);
                    if (lane == 0) { s_fin[0] = ql; s_fin[1] = qr; s_fin[2] = qn; s_fin[7] = (uint32_t)verdict; }
                }
                __syncthreads();
                quick = (int)s_fin[7];
                if (quick == 1) { left = s_fin[0]; right = s_fin[1]; rounds = s_fin[2]; }
                __syncthreads();     // everybody has read the outcome before the exact search may reuse the area
            }
        } else {
            if (emin == emax) {
                // every element has the same probability: the reference's loop never starts, the whole row ties
                left = __float_as_uint(pmin);
                right = left + 1u;
#pragma unroll
                for (int j = 0; j < LPT; j++) {
                    const int vl = j * NT + t;
                    eqk[j] = (vl < V4) ? (uint32_t)(((V4 - vl + kLanes - 1) >> 10) * 4) : 0u;
                }
                break;
            }
            // p = exp2f(x - max) / denom (sampling.cu:573-590) into the global scratch row
            // (one more pass of the copy pipeline over the row; the penalty stripes requested ahead are given up)
            list_left = __float_as_uint(pmin);
#pragma unroll
            for (int j = 0; j < LPT; j++) {
                const int vl = j * NT + t;
                n_row[j] = (vl < V4) ? ((V4 - vl + kLanes - 1) >> 10) * 4 : 0;
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            begin_pass(NC, 1, Yes(), Pen());
            auto write_p = [&](const int j, const int k, float4 v) {
                v.x = exp2f(v.x - mx) / denom; v.y = exp2f(v.y - mx) / denom;
                v.z = exp2f(v.z - mx) / denom; v.w = exp2f(v.w - mx) / denom;
                row.slab[(size_t)k * kLanes + j * NT + t] = v;
            };
            stream_x(write_p, [&](const int h, const int k, float4 (&v)[SL]) {
#pragma unroll
                for (int jj = 0; jj < SL; jj++) write_p(h * SL + jj, k, v[jj]);
            });
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        if (!whole && quick == 2) continue;
        const bool ok = (!whole && quick == 1) ? true : run_search(lane_eval, !whole, beta_p, !whole && use_cnt && nstrict > top_k, nstrict);
        const float thr_found = __uint_as_float(left);
        if (!whole) {
            if (!ok) continue;
            path = 0;
#pragma unroll
            for (int j = 0; j < LPT; j++)
                for (int i = 0; i < m_own[j]; i++) {
                    const float q = cand[i * kLanes + j * NT + t];
                    if (q == thr_found) eqk[j]++;
                    if (q > thr_found) { gtk[j]++; gtp[j] += q; }
                }
            break;
        }
        // recount on the whole row (sampling.cu:657-680)
#pragma unroll
        for (int j = 0; j < LPT; j++) {
            row.tg = j * NT + t;
            const int slots = (n_row[j] + 3) >> 2;
#pragma unroll 4
            for (int sidx = 0; sidx < slots; sidx++) {
                const float4 v = row.ld(sidx);
                const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    if (e[q] == thr_found) eqk[j]++;
                    if (e[q] > thr_found) { gtk[j]++; gtp[j] += e[q]; }
                }
            }
        }
        if (REP) begin_pass(K - 1, -1, No(), Yes());   // the update pass's first penalty stripes again
    }
    stamp(6);
    const bool early_exit = left < right - 1u;
    const float thr = __uint_as_float(left);

    // totals at the threshold (sampling.cu:657-680): lane 31 of a descending-offset scan holds the tree value
    float sgtp;
    uint32_t seqk, sgtk;
    if (path == 0 && !early_exit && quick != 1) {
        sgtp = conv_mass;
        sgtk = conv_cnt;
        seqk = conv_left_cnt - conv_cnt;
    } else {
        float m[NV];
        uint32_t c[4] = {0u, 0u, 0u, 0u}, cnt[4], d0, d1;
        float mass[4];
#pragma unroll
        for (int j = 0; j < LPT; j++) {
            m[j * 4 + 0] = gtp[j]; m[j * 4 + 1] = 0.f; m[j * 4 + 2] = 0.f; m[j * 4 + 3] = 0.f;
            c[0] += gtk[j];
            c[1] += eqk[j];
        }
        totals(m, c, 0u, 0u, cnt, mass, d0, d1);
        sgtp = mass[0];
        sgtk = cnt[0];
        seqk = cnt[1];
    }

    // ---- compensation factor for the boundary ties (sampling.cu:690-696, :903-908) ---------------------------
    float comp = 1.0f;
    if (seqk > 0) {
        comp = fminf(sanitize((top_p - sgtp) / (thr * seqk)), comp);
        if (use_cnt) comp = fminf(sanitize(float(top_k - sgtk) / seqk), comp);
        comp = fmaxf(comp, 0.0f);
    }

    // ---- lane pick (sampling.cu:699-723) -----------------------------------------------------------------------
    float incl[LPT];
    {
        float* box = box_of(phase);
#pragma unroll
        for (int j = 0; j < LPT; j++) {
            const float actual_p = gtp[j] + (thr * eqk[j]) * comp;
            incl[j] = warp_scan_desc(actual_p, lane);
            if (lane == 31) box[j * WPB + pw] = incl[j];
        }
        __syncthreads();
    }
    float sum_p, randp;
    {
        const float4* box4 = reinterpret_cast<const float4*>(box_of(phase));
        phase ^= 1;
        // sequential prefix over the 32 warp totals (sampling.cu:85-92); this thread needs the prefix before each of
        // its virtual warps j * WPB + pw, i.e. the running sum after warp w whenever w % WPB == pw - 1
        float before[LPT];
#pragma unroll
        for (int j = 0; j < LPT; j++) before[j] = 0.f;
        float s0 = 0.f;
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const float4 v = box4[q];
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const int w = q * 4 + r;
                s0 = (w == 0) ? e[r] : s0 + e[r];
                if ((w % WPB) == pw - 1 && w / WPB < LPT) before[w / WPB] = s0;             // prefix before warp w + 1, same j
                if (pw == 0 && (w % WPB) == WPB - 1 && w / WPB + 1 < LPT) before[w / WPB + 1] = s0;   // ... next j
            }
        }
        sum_p = s0;
        randp = sum_p * ux;
#pragma unroll
        for (int j = 0; j < LPT; j++) {
            const int vw = j * WPB + pw;
            const float pre_prev = before[j];
            const float cumu_p = (vw > 0) ? incl[j] + pre_prev : incl[j];
            const bool u = (randp <= cumu_p);
            bool u_prev = __shfl_up_sync(FULL, u, 1);
            if (lane == 0) u_prev = (vw > 0) ? (randp <= pre_prev) : false;
            // exactly one lane sees the 0 -> 1 transition (the scan is non-decreasing); with none the reference
            // keeps its initial value, lane 0
            if (u != u_prev) *s_idxt = j * NT + t;
        }
    }
    stamp(7);
    if (t == 0) {   // advance the stored RNG state by one 4-word block
        const uint4 nctr = ctr_next(rng.ctr);
        uint4* st = reinterpret_cast<uint4*>(p.states + (long long)b * RS_STATE_BYTES);
        st[0] = nctr;
        st[1] = philox4x32_10(nctr, rng.key_pos.x, rng.key_pos.y);
    }

    // ---- element pick inside the chosen lane (sampling.cu:725-751) ---------------------------------------------
    __syncthreads();
    const int idxt = *s_idxt;
    float oincl[LPT];
    int idn_of[LPT];
#pragma unroll
    for (int j = 0; j < LPT; j++) {
        const int vt = j * NT + t;   // thread index of the reference block
        const int idn = idxt * 4 + (vt >> 2) * 4 * kLanes + (vt & 3);
        float o0 = 0.f;
        if (idn < V) {
            const float x = scaled_logit(logit1(idn), rep ? prow[idn] : 0.f, rep, a_scale);
            o0 = exp2f(x - mx) / denom;
        }
        const float o = (o0 < thr) ? 0.f : (o0 == thr) ? (o0 * comp) : o0;
        oincl[j] = warp_scan_desc(o, lane);
        idn_of[j] = idn;
        if (lane == 31) s_wtot[vt >> 5] = oincl[j];
    }
    __syncthreads();
    float sum_o, rand2;
    {
        float opre[LPT];
#pragma unroll
        for (int j = 0; j < LPT; j++) opre[j] = 0.f;
        float s0 = 0.f;
        const float4* wt4 = reinterpret_cast<const float4*>(s_wtot);
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const float4 v = wt4[q];
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const int w = q * 4 + r;
                s0 = (w == 0) ? e[r] : s0 + e[r];
                if ((w % WPB) == pw - 1 && w / WPB < LPT) opre[w / WPB] = s0;
                if (pw == 0 && (w % WPB) == WPB - 1 && w / WPB + 1 < LPT) opre[w / WPB + 1] = s0;
            }
        }
        sum_o = s0;
        rand2 = sum_o * uy;
#pragma unroll
        for (int j = 0; j < LPT; j++) {
            const int vw = j * WPB + pw;
            const float cumu_o = (vw > 0) ? oincl[j] + opre[j] : oincl[j];
            const bool uo = (rand2 <= cumu_o);
            bool uo_prev = __shfl_up_sync(FULL, uo, 1);
            if (lane == 0) uo_prev = (vw > 0) ? (rand2 <= opre[j]) : false;
            if (uo != uo_prev) *s_token = (idn_of[j] < V) ? idn_of[j] : 0;
        }
    }
    __syncthreads();
    const int token = *s_token;
    stamp(8);
    if (t == 0) {
        p.out[b] = token;
        if (p.out_prob) {   // the sampled id's probability under the full softmax (its penalty is still the old one here)
            const float x = scaled_logit(logit1(token), rep ? prow[token] : 0.f, rep, a_scale);
            p.out_prob[b] = exp2f(x - mx) / denom;
        }
        if (p.out_kept) p.out_kept[b] = sum_p;
    }
    if (REP && p.out_prob) __syncthreads();     // nobody updates that penalty before it has been read

    // ---- penalties: decay everything, add the hit on the sampled id (sampling.cu:427-437); the old values come
    // through the copy pipeline, whose first stripes have been in flight since the second pass ended -------------
    if (rep) {
        int cslot = 0;
        auto stripe = [&](auto full_tag, const int k) {
            constexpr bool FULLK = decltype(full_tag)::value;
#pragma unroll
            for (int h = 0; h < NH; h++) {
            request(No(), Yes());
            wait_stage();
            const unsigned char* st = ring + (size_t)cslot * kStage;
#pragma unroll
            for (int jj = 0; jj < SL; jj++) {
                const int j = h * SL + jj;
                const int l = j * NT + t, i4 = k * kLanes + l;
                if (FULLK || tail_ok[j]) {
                    const float4 q4 = reinterpret_cast<const float4*>(st + kPart)[jj * NT + t];
                    float e[4] = {q4.x, q4.y, q4.z, q4.w};
                    if (i4 != (token >> 2)) {
#pragma unroll
                        for (int q = 0; q < 4; q++) e[q] = fmaf(e[q], p.decay, 0.f);
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const float old = e[q];
                            e[q] = fmaf(old, p.decay, (i4 * 4 + q != token) ? 0.f : (old == 0.f ? p.presence : p.repetition));
                        }
                    }
                    reinterpret_cast<float4*>(prow)[i4] = make_float4(e[0], e[1], e[2], e[3]);
                }
            }
            cslot = (cslot + 1 == D) ? 0 : cslot + 1;
            }
        };
        if (rem) stripe(TagRagged(), Kf);
        for (int k = Kf - 1; k >= 0; k--) stripe(TagFull(), k);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    stamp(9);
    if (t == 0 && p.dbg_trace) {
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
        tr.t_ns[0] = n_eval | ((uint32_t)quick << 16) | (ncand <= (uint32_t)kQuickCap ? 0x100000u : 0u);
        p.dbg_trace[b] = tr;
    }
}

// ------------------------------------------------------------------------------------------------ host side
// Shared memory of a row-CTA launch: fixed area, candidate lists (cap entries per virtual lane), copy stages, and the
// stripes that stay on chip between the passes.  The pipeline shape is a compile-time property of the four kernel
// instantiations:
// without penalties 4 stages of a whole stripe (16 KiB); with penalties 3 stages of 32 KiB when a row has an SM to itself
// (lanes_per_thread 2), and 5 stages of half a stripe (16 KiB: 8 of logits, 8 of penalties) when two rows share one.
static int rowcta_depth(bool rep, int lanes_per_thread) { return rep ? (lanes_per_thread == 2 ? 3 : 5) : 4; }
static int rowcta_parts(bool rep, int lanes_per_thread) { return (rep && lanes_per_thread == 4) ? 2 : 1; }

RowCtaPlan rowcta_plan(int V, bool rep, int sel_rank, int lanes_per_thread, int smem_budget) {
    RowCtaPlan pl;
    const int K = (V / 4 + kLanes - 1) / kLanes;
    pl.stage_bytes = (rep ? 2 : 1) * kStripeBytes / rowcta_parts(rep, lanes_per_thread);
    pl.cap = (sel_rank > 0) ? 6 : 0;
    pl.off_cand = kRowCtaFixedSmem;
    pl.off_ring = pl.off_cand + pl.cap * kLanes * 4;
    pl.depth = rowcta_depth(rep, lanes_per_thread);
    const int room = smem_budget - pl.off_ring - pl.depth * pl.stage_bytes;
    int keep = room / kStripeBytes;
    if (keep > K) keep = K;
    if (rowcta_parts(rep, lanes_per_thread) > 1) keep = 0;      // half-stripe stages keep nothing on chip
    pl.cached = keep < 0 ? 0 : keep;
    pl.off_cache = pl.off_ring + pl.depth * pl.stage_bytes;
    pl.smem_bytes = pl.off_cache + pl.cached * kStripeBytes;
    return pl;
}

template <int LPT, bool REP, int D, int NH, bool LOWP>
static int rowcta_launch_t(const Params& p, const RowCtaPlan& pl, cudaStream_t stream, int smem_optin, bool* attr_done, bool dependent) {
    auto kern = rowcta_kernel<LPT, REP, D, NH, LOWP>;
    if (!*attr_done) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin) != cudaSuccess) return RS_ERR_CUDA;
        *attr_done = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3((unsigned)p.B, 1, 1);
    cfg.blockDim = dim3(kLanes / LPT, 1, 1);
    cfg.dynamicSmemBytes = (size_t)pl.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel waits for its predecessor itself
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p, pl) == cudaSuccess ? RS_OK : RS_ERR_CUDA;
}

template <bool LOWP>
static int rowcta_launch_d(const Params& p, const RowCtaPlan& pl, int lanes_per_thread, bool rep, cudaStream_t stream, int smem_optin,
                           bool* attr_done, bool dependent) {
    if (lanes_per_thread == 2)
        return rep ? rowcta_launch_t<2, true, 3, 1, LOWP>(p, pl, stream, smem_optin, attr_done + 0, dependent)
                   : rowcta_launch_t<2, false, 4, 1, LOWP>(p, pl, stream, smem_optin, attr_done + 1, dependent);
    return rep ? rowcta_launch_t<4, true, 5, 2, LOWP>(p, pl, stream, smem_optin, attr_done + 2, dependent)
               : rowcta_launch_t<4, false, 4, 1, LOWP>(p, pl, stream, smem_optin, attr_done + 3, dependent);
}

int rowcta_launch(const Params& p, const RowCtaPlan& pl, int lanes_per_thread, cudaStream_t stream, int smem_optin, bool dependent) {
    static std::mutex mu;
    static bool attr_done[64][8] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return RS_ERR_CUDA;
    const bool rep = p.penalties != nullptr;
    if (pl.depth != rowcta_depth(rep, lanes_per_thread) || pl.smem_bytes > smem_optin) return RS_ERR_LIMIT;
    std::lock_guard<std::mutex> lk(mu);
    if (p.dtype == RS_DTYPE_F32) return rowcta_launch_d<false>(p, pl, lanes_per_thread, rep, stream, smem_optin, attr_done[dev], dependent);
    return rowcta_launch_d<true>(p, pl, lanes_per_thread, rep, stream, smem_optin, attr_done[dev] + 4, dependent);
}

}  // namespace rs
