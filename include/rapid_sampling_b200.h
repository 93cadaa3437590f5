/*
 * rapid_sampling_b200.h -- C ABI of the B200 (sm_100a) token sampler.
 *
 * Plain pointers and sizes only; every pointer named "device" must be device memory of the
 * CUDA device that is current on the calling thread.  `stream` is a cudaStream_t passed as
 * void* (NULL = the legacy default stream).  All sampling calls are asynchronous on `stream`.
 *
 * Each entry point names the reference interface it replaces (paths are those of the
 * reference project's files).
 */
#ifndef RAPID_SAMPLING_B200_H
#define RAPID_SAMPLING_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes (0 = success).  The reference throws std::invalid_argument for the first four
 * conditions (sampling.cu:452, :461, :467, :474 and :976, :986, :992, :999). */
enum {
    RS_OK = 0,
    RS_ERR_DTYPE = -1,       /* reserved for the tensor shim: logits are not fp32               */
    RS_ERR_VOCAB = -2,       /* V <= 0, V > 1048576 or V % 4 != 0                               */
    RS_ERR_BATCH = -3,       /* B <= 0 or T <= 0                                                */
    RS_ERR_TEMPERATURE = -4, /* temperature outside [0.001, 1000]                               */
    RS_ERR_POINTER = -5,     /* NULL or misaligned pointer (rows and states need 16 B alignment) */
    RS_ERR_WORKSPACE = -6,   /* workspace smaller than rs_workspace_bytes()                      */
    RS_ERR_CUDA = -7,        /* a CUDA runtime call failed; see rs_last_cuda_error()             */
    RS_ERR_TIMEOUT = -8,     /* device status: a bounded on-chip wait gave up                    */
    RS_ERR_LIMIT = -9,       /* size beyond what this entry point supports                       */
    RS_ERR_INTERNAL = -10    /* device status: an invariant of the cutoff search was violated    */
};

/* Bytes per row of the RNG state tensor: layout-compatible with curandStatePhilox4_32_10_t
 * (the reference's RAND, sampling.cu:9): ctr[4] | cached block[4] | key[2] | pos | 5 zero words. */
#define RS_STATE_BYTES 64

/* Per-row values captured by rs_sample_debug(); all are the kernel's own fp32/u32 values. */
typedef struct rs_trace {
    float maxu, denom, pmin, pmax, threshold, comp, sgtp, sum_p, randp, sum_o, rand2;
    uint32_t left, seqk, sgtk, rounds, idxt, early_exit, rnd[4];
    int32_t token;
    uint32_t path;   /* 0 = cutoff found on the candidate list, 1 = whole-row search */
    uint32_t ncand;  /* elements on the candidate list */
    uint32_t t_ns[10]; /* ns since kernel entry of the owner CTA's thread 0 at: 1 row resident, 2 pass 1, 3 exchange,
                          4 pass 2, 5 exchange, 6 search+recount, 7 lane pick, 8 element pick, 9 end.  Entry 0: rounds of
                          the search that needed block-wide sums (bits 0-15); the one-CTA-per-row kernel adds the outcome
                          of its one-warp integer search in bits 16-19 (1 settled, 2 list too short, 0 undecided or not tried) */
} rs_trace;

/*
 * Replaces setup_rand(seed, B) (sampling.cpp:6, sampling.cu:136-144): fills B states so that
 * row b is subsequence (first_row + b) of `seed`, offset 0.  The reference always uses
 * first_row = 0; a batch shard passes its global row offset so that sharded and unsharded runs
 * draw the same numbers.  states_device: B * RS_STATE_BYTES bytes, 16-byte aligned.
 */
int rs_setup_rand(void* states_device, uint64_t seed, int64_t B, int64_t first_row, void* stream);

/* Device scratch a call with this shape may need, plus a status word.  Never 0.  Batches that fit on chip at
 * once need only the status word (256 bytes); larger batches and rows too large for on-chip storage run the
 * streaming variant, whose fallback uses a B*V fp32 scratch (the counterpart of the reference's `probs`,
 * sampling.cu:488, :1014).  A call given less than this runs on chip when the row fits, else fails with
 * RS_ERR_WORKSPACE. */
size_t rs_workspace_bytes(int64_t B, int64_t V);

/*
 * Replaces batch_sampling_temperature_topk_topp (sampling.cpp:8, sampling.cu:968-1044) when
 * penalties_device == NULL, and batch_sampling_repetition_temperature_topk_topp
 * (sampling.cpp:7, sampling.cu:440-515) otherwise.
 *
 * logits_device   fp32 (B, T, V) contiguous; only position T-1 of each row is read
 *                 (sampling.cu:176, :202).  Pass T = 1 for (B, V) / (V,) input.
 * penalties_device fp32 (B, V), updated in place with decay and the hit (sampling.cu:427-437), or NULL.
 * states_device   B * RS_STATE_BYTES bytes; each row consumes one 4-word block (sampling.cu:383).
 * out_device      int32[B] sampled ids (the reference returns an int32 tensor, sampling.cu:498, :1024).
 * temperature, top_k, top_p  checked and remapped exactly as sampling.cu:474-486 / :999-1010.
 * workspace_device / workspace_bytes  at least rs_workspace_bytes(B, V), 256-byte aligned.
 */
int rs_sample(const float* logits_device, int64_t B, int64_t T, int64_t V, float* penalties_device,
              void* states_device, int32_t* out_device, double temperature, int64_t top_k, double top_p,
              double presence_penalty, double repetition_penalty, double penalty_decay,
              void* workspace_device, size_t workspace_bytes, void* stream);

/* Same call, additionally writing the probabilities the cutoff search ran on (fp32 (B, V), may be
 * NULL) and one rs_trace per row (may be NULL).  No reference counterpart: test instrumentation
 * of the same kernels (the reference's equivalents are its commented-out printf macros,
 * sampling.cu:146-147). */
int rs_sample_debug(const float* logits_device, int64_t B, int64_t T, int64_t V, float* penalties_device,
                    void* states_device, int32_t* out_device, double temperature, int64_t top_k, double top_p,
                    double presence_penalty, double repetition_penalty, double penalty_decay,
                    void* workspace_device, size_t workspace_bytes, void* stream,
                    float* probs_device, rs_trace* trace_device);

/*
 * rs_sample / rs_sample_debug for logits stored as fp32, fp16 or bf16.  The reference accepts fp32 only and throws
 * for anything else (sampling.cu:452, :976); a model head usually emits 16-bit logits, so this entry point reads
 * them directly (half the HBM bytes per row) and widens each value exactly to fp32 before the first operation --
 * the result is bit-identical to calling the fp32 entry point on `logits.float()`.  Rows need 8-byte alignment
 * for the 16-bit types.  probs_device / trace_device may be NULL.
 */
enum { RS_DTYPE_F32 = 0, RS_DTYPE_F16 = 1, RS_DTYPE_BF16 = 2 };
int rs_sample_typed(const void* logits_device, int32_t logits_dtype, int64_t B, int64_t T, int64_t V,
                    float* penalties_device, void* states_device, int32_t* out_device, double temperature, int64_t top_k,
                    double top_p, double presence_penalty, double repetition_penalty, double penalty_decay,
                    void* workspace_device, size_t workspace_bytes, void* stream, float* probs_device,
                    rs_trace* trace_device);

/*
 * Per-row parameters.  No counterpart in the reference, whose host functions take one scalar temperature / top_k /
 * top_p per call (sampling.cpp:2-3); a serving batch mixes requests with different settings.
 * temperature_device / top_k_device / top_p_device are device arrays of B values (float32 / int32 / float32);
 * a NULL array stands for the neutral value in every row (temperature 1, top_k -1, top_p 1).  Each row is
 * sampled exactly as a one-row call of rs_sample_typed with that row's values would sample it (same checks and
 * remaps, sampling.cu:458-486, applied on the device; same ids, states and penalties), except that a temperature
 * outside [0.001, 1000] cannot be refused by a call that does not read the array: such a row is sampled at
 * temperature 1 and the device status word is set to RS_ERR_TEMPERATURE (rs_device_status).
 * out_prob_device (optional, B floats): the sampled id's probability under the full softmax of the scaled /
 * penalised row.  out_kept_mass_device (optional, B floats): the probability mass of the kept set the id was
 * drawn from (boundary ties counted with their fractional weight, sampling.cu:690-696).
 * The workspace needs rs_rows_workspace_bytes(B, V) bytes, zero-initialised once, 256-byte aligned.
 */
size_t rs_rows_workspace_bytes(int64_t B, int64_t V);
int rs_sample_rows(const void* logits_device, int32_t logits_dtype, int64_t B, int64_t T, int64_t V,
                   float* penalties_device, void* states_device, int32_t* out_device, const float* temperature_device,
                   const int32_t* top_k_device, const float* top_p_device, double presence_penalty,
                   double repetition_penalty, double penalty_decay, float* out_prob_device, float* out_kept_mass_device,
                   void* workspace_device, size_t workspace_bytes, void* stream);

/*
 * Host-buffer convenience around rs_sample for callers that hold logits in (pinned) host memory:
 * copies logits[:, T-1, :] to `staging_device` (B*V floats), samples, copies the ids back to
 * out_host and synchronises `stream`.  Penalties and states stay on the device.
 */
int rs_sample_host(const float* logits_host, int64_t B, int64_t T, int64_t V, float* penalties_device,
                   void* states_device, int32_t* out_host, double temperature, int64_t top_k, double top_p,
                   double presence_penalty, double repetition_penalty, double penalty_decay,
                   float* staging_device, int32_t* out_device, void* workspace_device, size_t workspace_bytes,
                   void* stream);

/*
 * Sampling for callers that cannot allocate device memory.  No counterpart in the reference (its host
 * functions allocate a scratch tensor on every call, sampling.cu:488, :1014).
 *
 * Who needs it: a serving process that gave all of HBM to its own arena at start-up, so that cudaMalloc has
 * nothing left to hand out; and a latency-critical decode loop that must not enter an allocator which may
 * synchronise the device.  Same arguments and results as rs_sample, but without a workspace: the kernel's
 * scratch rows live in a fixed array inside the library image (16 MiB + 256 B, held by every GPU that loads
 * the library until the process exits), and the call performs no cudaMalloc, cudaFree or other allocation.
 *
 * Limits and rules:
 *  - B * V must not exceed RS_STATIC_SCRATCH_FLOATS, otherwise RS_ERR_LIMIT is returned and nothing runs.
 *  - The first call on each device looks up the array's device address (and clears its status word, on the
 *    call's stream); make that first call before any stream capture begins.  rs_device_status(NULL, stream)
 *    reads that status word.
 *  - All calls on a device share the one array, which keeps whatever the previous call left in it (the kernel
 *    overwrites what it reads, only the status word relies on the initial clearing).  Two calls that overlap
 *    on the GPU (different streams) race on it: keep calls to this entry point on one stream, or order them.
 *  - It always runs the global-scratch-row variant of the kernel, so it is slower than rs_sample for rows that
 *    would fit on chip; ids, states and penalties are identical to rs_sample's.
 */
#define RS_STATIC_SCRATCH_FLOATS 4194304
int rs_sample_static_scratch(const float* logits_device, int64_t B, int64_t T, int64_t V, float* penalties_device,
                             void* states_device, int32_t* out_device, double temperature, int64_t top_k, double top_p,
                             double presence_penalty, double repetition_penalty, double penalty_decay, void* stream);

/*
 * Vocab-parallel sampling: every GPU holds V_local = V_global / world columns of each row, as a tensor-parallel
 * lm_head produces them.  No counterpart in the reference (single GPU only, no collective in sampling.cu); the
 * sampling semantics are those of its kernels evaluated on the union of the shards.  The call is cut into
 * stages; between two stages the host reduces a small region of the workspace across ranks (NCCL):
 *
 *   stage            then reduce (op) over ranks             workspace region (offsets from rs_vp_layout, floats)
 *   RS_VP_MAX        MAX   B floats                          [0] row maxima
 *   RS_VP_SUM        SUM   B floats                          [1] softmax denominators
 *   RS_VP_ROUND r    SUM   B*15*2 floats (round r's slice)   [2] + r*B*30: counts and masses at 15 pivots, r = 0..7
 *   RS_VP_TALLY      SUM   B*4 floats                        [3] count above / mass above / ties at the threshold
 *   RS_VP_WEIGHT     SUM   B*world floats                    [4] kept weight per shard (owner election)
 *   RS_VP_PICK       MAX   B int32                           [5] sampled id + 1 (0 from non-owners)
 *   RS_VP_PENALTY    --                                      updates this shard's penalty columns in place
 *
 * Every rank holds a replica of `states` (same seed) and advances it identically.  Results are deterministic and
 * identical on all ranks; they are not bit-identical to the single-GPU kernel (different summation order).
 */
#define RS_VP_ROUNDS 8
enum { RS_VP_MAX = 0, RS_VP_SUM = 1, RS_VP_ROUND = 2, RS_VP_TALLY = 3, RS_VP_WEIGHT = 4, RS_VP_PICK = 5, RS_VP_PENALTY = 6,
       /* fast protocol (3 collectives): every shard extracts a short candidate list, the lists are all-gathered and every
        * rank finishes the row on the union.  Order: VPF_MAX, VPF_SUM (denominator + octave histogram of the large
        * elements), VPF_EXTRACT (bound chosen from the reduced histogram), VPF_COMPACT, all-gather, VPF_FINISH.
        * Regions from rs_vp_fast_layout (floats): [0] stat1 B*S (all-reduce MAX),
        * [1] stat2 B*S*[10] (all-reduce SUM), [2] send list B*Lmax*2 + [3] send counts B (all-gather into [4] and [5]),
        * [6] ids + 1 (int32 B), [7] valid flags (int32 B; a 0 means: repeat the call with the staged protocol),
        * [8] = S, [9] = Lmax.  RS_VP_PENALTY with round = 1 applies the fast protocol's ids. */
       RS_VPF_MAX = 10, RS_VPF_SUM = 11, RS_VPF_COMPACT = 12, RS_VPF_FINISH = 13, RS_VPF_ADVANCE = 14, RS_VPF_EXTRACT = 15 };
typedef struct rs_vp_call {
    const float* logits;      /* device, (B, T, V_local) contiguous: this rank's columns; position T-1 is read   */
    float* penalties;         /* device, (B, V_local) or NULL                                                    */
    void* states;             /* device, B * RS_STATE_BYTES, a replica of the same states on every rank          */
    void* workspace;          /* device, rs_vp_workspace_bytes(B, world) bytes                                   */
    void* stream;             /* cudaStream_t                                                                    */
    int64_t B, T, V_local, V_global, col0;   /* col0 = global index of this shard's first column               */
    int64_t top_k;
    double temperature, top_p, presence_penalty, repetition_penalty, penalty_decay;
    int32_t rank, world;
} rs_vp_call;
size_t rs_vp_workspace_bytes(int64_t B, int32_t world);
int rs_vp_layout(int64_t B, int32_t world, int64_t offsets_floats[6]);
int rs_vp_fast_layout(int64_t B, int64_t V_local, int32_t world, int64_t offsets_floats[11]);
int rs_vp_stage(const rs_vp_call* call, int32_t stage, int32_t round);

/*
 * lm_head epilogue hook for the vocab-parallel fast protocol.  No counterpart in the reference (it allocates, launches
 * and reads a finished logits tensor per call, sampling.cu:488, :498, :1014, :1024).  A tensor-parallel lm_head produces
 * this rank's (B, V_local) logits tile by tile; instead of a separate pass over the finished shard for the row maxima
 * (stage RS_VPF_MAX), the producer hands every tile over as soon as it exists:
 *
 *   rs_vp_tile_begin(call)                                  once per sampling call, before the first tile
 *   rs_vp_tile_max(call, tile, ld, col_begin, ncols)        per tile, any order, any tile width; `tile` points at row 0
 *                                                           of the tile (position T-1), rows `ld` elements apart,
 *                                                           holding local columns [col_begin, col_begin + ncols)
 *   all-reduce MAX of region [0] of rs_vp_fast_layout, then RS_VPF_SUM, RS_VPF_EXTRACT, ... as usual
 *
 * Both calls are asynchronous on call->stream, use only the preallocated workspace and allocate nothing.  The fold is an
 * atomic maximum, so the result does not depend on the order of the tiles.  call->penalties (if any) must be final when
 * a tile is handed over; call->logits is not read by these two calls (the later stages read it, so the tiles must end up
 * in that buffer).
 */
int rs_vp_tile_begin(const rs_vp_call* call);
int rs_vp_tile_max(const rs_vp_call* call, const float* tile_device, int64_t ld, int64_t col_begin, int64_t ncols);

/*
 * Device status word.  The kernels never trap: a condition they cannot report through a return code is written to
 * the first int32 of the workspace, which stays set until it is cleared.  Values: RS_OK; RS_ERR_TIMEOUT (a bounded
 * on-chip wait gave up: the rows of the CTAs that saw it report id -1 and leave their RNG state and penalties
 * untouched; other rows of the call are unaffected); RS_ERR_TEMPERATURE (rs_sample_rows: some row's temperature
 * lay outside [0.001, 1000] and was sampled at 1).  No reference counterpart: the reference checks nothing after
 * a launch (sampling.cu:500-515).
 *
 * rs_device_status reads the word (synchronises `stream`); rs_clear_status zeroes it on `stream`.  For both,
 * workspace_device == NULL names the status word of rs_sample_static_scratch's built-in array on the current device.
 */
int rs_device_status(void* workspace_device, void* stream);
int rs_clear_status(void* workspace_device, void* stream);

/*
 * Optional host mirror of the status word for the current device: `host_word` must be a 4-byte word of pinned,
 * device-accessible host memory (cudaHostAlloc / cudaHostRegister; NULL removes the mirror).  Kernels launched
 * afterwards store a non-zero status there as well, so a host can notice a failure by reading its own memory,
 * without a copy or a synchronisation.  The caller owns the word and clears it.
 */
int rs_set_status_mirror(int* host_word);

/* Poll limit of the kernels' bounded waits (each poll blocks for a short hardware-defined time).  0 only queries.
 * Returns the previous limit.  The default (about four million polls) is far beyond any legitimate wait. */
uint32_t rs_set_wait_polls(uint32_t polls);

/*
 * Test instrumentation for the failure path, no reference counterpart: launches one CTA that waits with the given
 * poll limit (1..4096) on a barrier nothing will ever complete -- no copy or remote store is in flight -- and
 * reports the expiry as the sampler does: RS_ERR_TIMEOUT in the status word of `workspace_device` (and the
 * mirror).  The GPU context stays usable.
 */
int rs_selftest_bounded_wait(void* workspace_device, uint32_t polls, void* stream);

/* The sampler kernels are launched with programmatic stream serialization: a kernel may be scheduled while its
 * predecessor in the stream still runs, and waits on the device (before it touches any global memory) until that
 * predecessor is complete and its writes are visible.  Between back-to-back sampler calls this hides the launch latency.
 * Only grids of at most half the GPU's SMs are launched this way (larger ones are better placed on an empty GPU).
 * 0 switches to ordinary launches, 1 (default) back; any other value only reads.  Returns the previous setting. */
int rs_set_dependent_launch(int on);

/* Forces the thread-block-cluster width (1, 2, 4, 8 or 16) used per row; 0 restores the automatic
 * choice.  Benchmarking aid; returns the previous value. */
int rs_set_cluster_override(int cluster_ctas);

/* Strategy override: 0 = automatic, 1 = always search the whole row (no candidate shortcut), 2 = always the
 * streaming cluster variant, 3 = always the on-chip cluster variant when the row fits, 4 = always one CTA per row
 * (calls with a full-size workspace; other calls keep the automatic choice), 5 = as 4 and 6 = as 0, but with the exact
 * search on fp32 sums only (no one-warp search on integer masses first).  Results are identical; testing / benchmarking
 * aid.  Returns the previous value. */
int rs_set_path_override(int mode);

/* Number of sampler kernels launched through this library since it was loaded. */
uint64_t rs_kernel_launch_count(void);

const char* rs_status_string(int status);
const char* rs_last_cuda_error(void);
const char* rs_version(void);

#ifdef __cplusplus
}
#endif
#endif /* RAPID_SAMPLING_B200_H */
