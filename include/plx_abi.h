/*
 * plx_abi.h -- C ABI of libplx_sm100.so: the Parallax attention hot path
 * (dense causal training forward/backward, packed variable-length training,
 * single-token KV-cache decode) as hand-written CUDA for NVIDIA B200 (sm_100a).
 *
 * The upstream project (Yifei-Zuo/Parallax) is pure Python: its "plugin
 * boundary" is a set of Python functions that JIT-compile Triton / CuTeDSL
 * kernels.  Each entry point below names the upstream function whose device
 * work it replaces (paths are relative to the upstream checkout).
 *
 * Conventions
 *   - plain C types only; every pointer named q/r/k/v/o/... is a DEVICE pointer;
 *   - a function returns PLX_OK (0) or a negative PLX_ERR_* code and never throws;
 *   - no function allocates device memory, synchronises or changes device
 *     state unless its comment says otherwise; kernels are enqueued on `stream`;
 *   - the caller owns all buffers, including scratch ("workspace");
 *   - results are deterministic: no floating-point atomics on outputs.
 */
#ifndef PLX_ABI_H
#define PLX_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PLX_ABI_VERSION 2

/* cudaStream_t without pulling in the CUDA headers */
typedef struct CUstream_st *plx_stream_t;

enum plx_status {
    PLX_OK = 0,
    PLX_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, inconsistent heads ... */
    PLX_ERR_UNSUPPORTED = -2,  /* head_dim / dtype / shape this build has no kernel for  */
    PLX_ERR_LAUNCH = -3,       /* CUDA reported an error at launch                        */
    PLX_ERR_WORKSPACE = -4,    /* workspace missing or smaller than required              */
    PLX_ERR_DEVICE = -5,       /* current device is not sm_100                            */
    PLX_ERR_STATIC_SCRATCH = -6 /* problem needs more than the built-in scratch of plx_decode_static */
};

enum plx_dtype { PLX_BF16 = 0, PLX_FP16 = 1 };

/* ------------------------------------------------------------------------- *
 * Training (dense and packed).
 *
 * q, r, o, barv, grad_o, dq, dr share one layout ("q-like"), k, v, dk, dv
 * another ("kv-like"); both are given as ELEMENT strides for (batch, head,
 * token), the head_dim axis is contiguous.  This covers the upstream dense
 * layout (B, H, L, D) [parallax/triton/parallax_train.py:1039-1087] and the
 * heads-last packed layout (1, T, H, D) [parallax/triton/parallax_varlen.py:738-788].
 * The statistics d1, bart, m are fp32 with their own (batch, head, token) strides.
 *
 * Masking: query i of a sequence with len_q queries and len_k keys sits at
 * absolute position i + (len_k - len_q); it sees key j iff j <= pos and, for
 * window_left >= 0, j >= pos - window_left + 1  [parallax/reference.py:64-73].
 *
 * Packed input: cu_seqlens (device, int32, n_seqs + 1 entries, cu[0] = 0) splits
 * the token axis into independent causal sequences; batch must be 1 and
 * len_q == len_k == total tokens.  cu_seqlens == NULL means dense.
 * ------------------------------------------------------------------------- */
typedef struct plx_train_problem {
    int32_t dtype;        /* plx_dtype of q, r, k, v, o, barv and all gradients */
    int32_t batch;
    int32_t heads_q;
    int32_t heads_kv;     /* heads_q % heads_kv == 0 (grouped-query attention) */
    int32_t len_q;
    int32_t len_k;
    int32_t head_dim;     /* 64 or 128 */
    int32_t window_left;  /* -1 = no sliding window */
    float qk_scale;       /* multiplies q.k only; r.k is never scaled */
    int32_t n_seqs;       /* packed: number of sequences; dense: 0 */
    int64_t q_stride_b, q_stride_h, q_stride_t;
    int64_t kv_stride_b, kv_stride_h, kv_stride_t;
    int64_t st_stride_b, st_stride_h, st_stride_t;
    const int32_t *cu_seqlens;
} plx_train_problem;

/* Bytes of scratch plx_train_bwd needs (per-row backward statistics).
 * Replaces the `t` / `b` allocations of parallax_bwd
 * [parallax/triton/parallax_train.py:936-938]. */
int plx_train_workspace_bytes(const plx_train_problem *p, size_t *bytes);

/* Forward: o and barv (dtype), d1, bart, m (fp32; m in base-2 units of the
 * scaled logits, d1 un-normalised, bart = d2/d1, barv = O1/d1).
 * Replaces parallax_fwd + _fwd_kernel [parallax/triton/parallax_train.py:255-313, 42-252]
 * and parallax_varlen_fwd + parallel_parallax_fwd_kernel
 * [parallax/triton/parallax_varlen.py:637-659, 25-196]. */
int plx_train_fwd(const plx_train_problem *p, const void *q, const void *r, const void *k,
                  const void *v, void *o, void *barv, float *d1, float *bart, float *m,
                  plx_stream_t stream);

/* Backward: dq, dr (q-like) and dk, dv (kv-like, already summed over the q heads
 * of a group).  `workspace` must hold plx_train_workspace_bytes() bytes.
 * Replaces parallax_bwd and its three kernels
 * [parallax/triton/parallax_train.py:892-1006, 336-392, 395-612, 615-889] and
 * parallax_varlen_bwd [parallax/triton/parallax_varlen.py:662-711, 199-634],
 * including the torch-side GQA fold [parallax/triton/parallax_train.py:998-1005]. */
int plx_train_bwd(const plx_train_problem *p, const void *q, const void *r, const void *k,
                  const void *v, const void *o, const void *barv, const float *d1,
                  const float *bart, const float *m, const void *grad_o, void *dq, void *dr,
                  void *dk, void *dv, void *workspace, size_t workspace_bytes,
                  plx_stream_t stream);

/* The backward is three kernels, as upstream: row statistics t = go.o, b = go.barv
 * (_bwd_preprocess_kernel, parallax/triton/parallax_train.py:336-392), dq/dr
 * (_bwd_rq_kernel, :395-612) and dk/dv (_bwd_kv_kernel, :615-889).  `stages` is
 * a mask of PLX_BWD_* selecting which of them to enqueue (statistics must have
 * run on the same workspace before the other two); plx_train_bwd == PLX_BWD_ALL. */
enum plx_bwd_stage { PLX_BWD_STATS = 1, PLX_BWD_DQR = 2, PLX_BWD_DKV = 4, PLX_BWD_ALL = 7 };
int plx_train_bwd_stages(const plx_train_problem *p, int32_t stages, const void *q, const void *r,
                         const void *k, const void *v, const void *o, const void *barv,
                         const float *d1, const float *bart, const float *m, const void *grad_o,
                         void *dq, void *dr, void *dk, void *dv, void *workspace,
                         size_t workspace_bytes, plx_stream_t stream);

/* ------------------------------------------------------------------------- *
 * Decode: one query token per sequence against a KV cache.
 *
 * q, r, out: (batch, heads_q, head_dim) contiguous.  k, v: (batch, cache_len,
 * heads_kv, head_dim) addressed by element strides.  Active key range of batch
 * row b, in GLOBAL key positions (kv_offset is the global position of this
 * buffer's key 0, total_len the global cache length; 0 and cache_len for an
 * unsharded cache):
 *     hi = seqused_k ? clamp(seqused_k[b], 1, total_len) : total_len
 *     lo = max(cache_start ? cache_start[b] : 0, window_left >= 0 ? hi - window_left : 0, 0)
 * [parallax/triton/parallax_decode.py:48-54, parallax/cute/parallax_decode.py:367-369].
 * The kernel splits [lo, hi) over n_splits warps per (batch, head) and the last
 * warp to finish merges the partial states, so one launch produces `out`.  With
 * more than PLX_DECODE_GROUP_MIN splits the merge has two levels: the last warp
 * of every group of PLX_DECODE_GROUP splits merges its group, the last group the
 * group results.
 *
 * Workspace: plx_decode_workspace_bytes() bytes, ZERO-FILLED ONCE by the caller
 * before its first use (it holds arrival counters that the kernel resets itself).
 * Two launches that may overlap on the device must not share a workspace.
 * ------------------------------------------------------------------------- */
typedef struct plx_decode_problem {
    int32_t dtype;
    int32_t batch;
    int32_t heads_q;
    int32_t heads_kv;
    int32_t cache_len;    /* keys held by this k/v buffer */
    int32_t head_dim;     /* 64 or 128 */
    int32_t window_left;  /* -1 = off */
    int32_t n_splits;     /* 1 .. PLX_DECODE_MAX_SPLITS, see plx_decode_choose_splits */
    float qk_scale;
    int32_t kv_offset;    /* global position of key 0 of this buffer (KV-sharded decode) */
    int32_t total_len;    /* global cache length; 0 means cache_len */
    int64_t kv_stride_b, kv_stride_t, kv_stride_h;
    /* Paged cache (page_table != NULL; NULL = dense): k, v are (num_pages, page_size, heads_kv, head_dim),
     * kv_stride_b is the stride between PAGES, and key j of batch row b is row j % page_size of page
     * page_table[b * pages_per_seq + j / page_size].  page_size is a power of two; cache_len is the
     * logical ceiling (at most pages_per_seq * page_size).  Only entries that cover keys below the
     * active length of a row are read, so the tail of a row of the table may hold anything.  The
     * layout is flash_attn_with_kvcache's block table, which the upstream front end names but does
     * not implement [parallax/cute/parallax_decode.py:1578-1580, 1627-1632]. */
    const int32_t *page_table;   /* device, int32 */
    int32_t page_size;
    int32_t pages_per_seq;
} plx_decode_problem;

#define PLX_DECODE_MAX_SPLITS 256   /* upper bound of plx_decode_problem.n_splits */
/* With at most this many (batch, q head) pairs (heads_q == heads_kv), at most 2^19 / pairs keys in the
 * cache (or the window) and a split count that is a multiple of 8, eight adjacent splits share a CTA and
 * merge in shared memory ("split groups"): the latency-bound small-batch arrangement.
 * plx_decode_choose_splits picks such counts there. */
#define PLX_DECODE_SPLIT_GROUP_MAX_BH 64
#define PLX_DECODE_GROUP 16         /* splits merged by one warp at the first level */
#define PLX_DECODE_GROUP_MIN 32     /* up to this many splits are merged in one level */
/* Number of first-level groups (0 = single-level merge). */
#define PLX_DECODE_GROUPS(n_splits) \
    ((n_splits) > PLX_DECODE_GROUP_MIN ? ((n_splits) + PLX_DECODE_GROUP - 1) / PLX_DECODE_GROUP : 0)
/* Size of one partial-state record in floats: m, d1, d2, pad, O1[D], O2[D]. */
#define PLX_DECODE_PART_FLOATS(head_dim) (2 * (head_dim) + 4)
/* Workspace = batch * heads_q * ((n_splits + groups) records + (1 + groups) int32 counters). */

/* Split count for a (batch * heads_q) x n_keys problem on a device with
 * `sm_count` SMs.  Pure host arithmetic.  Plays the role of
 * _choose_num_k_splits [parallax/cute/parallax_decode.py:1347-1359]. */
int plx_decode_choose_splits(int32_t batch, int32_t heads_q, int32_t n_keys, int32_t sm_count);
/* The same for grouped-query shapes (heads_q > heads_kv), which run a different kernel
 * (q heads of a group packed into the M dimension of tensor-core MMAs, as upstream's
 * GQA packing [parallax/cute/parallax_decode.py:149-154]); falls back to the function
 * above when heads_q == heads_kv. */
int plx_decode_choose_splits_gqa(int32_t batch, int32_t heads_q, int32_t heads_kv, int32_t n_keys,
                                 int32_t sm_count);

int plx_decode_workspace_bytes(const plx_decode_problem *p, size_t *bytes);

/* out = Parallax decode.  seqused_k and cache_start are device int32 (batch,)
 * arrays or NULL.  Replaces parallax.triton.parallax_decode + its kernel
 * [parallax/triton/parallax_decode.py:100-148, 20-97] and the CuTeDSL path
 * _decode_core / ParallaxDecodePersistentSplit
 * [parallax/cute/parallax_decode.py:1408-1522, 135-1136]. */
int plx_decode(const plx_decode_problem *p, const void *q, const void *r, const void *k,
               const void *v, void *out, const int32_t *seqused_k, const int32_t *cache_start,
               void *workspace, size_t workspace_bytes, plx_stream_t stream);

/* plx_decode for callers that cannot allocate device memory.  (No counterpart in
 * the reference: upstream always allocates its split-KV workspace with torch.)
 *
 * Who needs it: code that is handed inputs and an output buffer but no allocator
 * -- an enqueue-style plugin callback inside a serving runtime that owns all device
 * memory, or a latency-critical decode loop in which cudaMalloc's device-wide
 * synchronisation is not affordable -- and therefore cannot provide the
 * `workspace` that plx_decode wants.  Here the split-KV scratch is a fixed array
 * of PLX_DECODE_STATIC_SCRATCH_BYTES bytes that lives inside the library's device
 * image: every GPU on which the library's kernels are loaded holds those bytes
 * until the process exits.  The function calls no cudaMalloc / cudaFree and no
 * allocating library routine; it only enqueues a small memset and the kernel.
 *
 *   - A problem whose scratch (plx_decode_workspace_bytes) exceeds the array is
 *     refused with PLX_ERR_STATIC_SCRATCH before anything is enqueued; lower
 *     n_splits or use plx_decode with your own workspace.
 *   - The first call on each device looks up the array's device address (with that
 *     device current); make that first call outside any stream capture.
 *   - All calls on a device share the one array.  Each call clears the arrival
 *     counters it is about to use, so a call never depends on what an earlier call
 *     (of any shape) left behind -- but two calls that can overlap on the GPU
 *     (different streams, no dependency) race on it and give wrong answers. */
#define PLX_DECODE_STATIC_SCRATCH_BYTES (4u << 20)
int plx_decode_static(const plx_decode_problem *p, const void *q, const void *r, const void *k,
                      const void *v, void *out, const int32_t *seqused_k,
                      const int32_t *cache_start, plx_stream_t stream);

/* Same sweep, but instead of `out` it writes ONE un-normalised partial state
 * per (batch, head) to `part` (batch * heads_q records of
 * PLX_DECODE_PART_FLOATS floats; m is the base-2 maximum of the scaled logits,
 * -inf for an empty range).  Used when the key axis is sharded over GPUs.  The
 * partial-state quintuple is that of the upstream split-KV workspace
 * [parallax/cute/parallax_decode.py:1368-1405]. */
int plx_decode_partial(const plx_decode_problem *p, const void *q, const void *r, const void *k,
                       const void *v, float *part, const int32_t *seqused_k,
                       const int32_t *cache_start, void *workspace, size_t workspace_bytes,
                       plx_stream_t stream);

/* Merge n_parts partial-state arrays (part s, record i at
 * parts + (s * n_records + i) * PLX_DECODE_PART_FLOATS) and finalise
 * out = (1 + d2/d1) * O1/d1 - O2/d1  [parallax/cute/parallax_decode.py:1107-1136].
 * n_records = batch * heads_q; out has n_records * head_dim elements of `dtype`. */
int plx_decode_merge(const float *parts, int32_t n_parts, int32_t n_records, int32_t head_dim,
                     int32_t dtype, void *out, plx_stream_t stream);

/* Exchange + merge in ONE kernel over peer memory, for ranks of one node whose GPUs can address each
 * other (NVLink): replaces "all-gather the partial records, then plx_decode_merge".  (No counterpart in
 * the reference, which is single-GPU.)
 *
 * Every rank owns an inbox of plx_decode_exchange_bytes() bytes, ZERO-FILLED ONCE, that every rank has
 * mapped; `inbox[r]` is rank r's inbox as addressed from THIS process (own rank included).  A call
 * stores this rank's `part` (n_records records, as plx_decode_partial wrote them) into every inbox,
 * waits for the other ranks' records of the same step and writes the merged, finalised `out`
 * (n_records * head_dim elements) on every rank.  The step count is kept in the inbox by the kernel
 * itself, so a captured launch can be replayed; all ranks must make the same sequence of calls on an
 * inbox.  The wait is bounded (`wait_ms`): when rank r never delivers record i, the kernel sets bit r of
 * `*status`, reports (40 + r) through plx_device_error, writes NaN into row i of `out` and still advances
 * the step count, so the ranks stay in step for the next call.  Peer stores and loads only: no TMA, no
 * multicast. */
#define PLX_EXCHANGE_MAX_RANKS 16
#define PLX_EXCHANGE_DEFAULT_WAIT_MS 2000
typedef struct plx_exchange {
    int32_t world, rank;      /* ranks sharing the inbox mapping, this rank */
    int32_t n_records;        /* batch * heads_q */
    int32_t head_dim, dtype;  /* of `out` */
    uint32_t wait_ms;         /* bound of the wait for the peers; 0 = PLX_EXCHANGE_DEFAULT_WAIT_MS */
    int32_t *status;          /* device int32, caller-owned and zeroed, or NULL: bit r = rank r timed out */
    void *inbox[PLX_EXCHANGE_MAX_RANKS];
} plx_exchange;
size_t plx_decode_exchange_bytes(int32_t world, int32_t n_records, int32_t head_dim);
int plx_decode_exchange_merge(const plx_exchange *x, const float *part, void *out, plx_stream_t stream);

/* The whole KV-sharded step as ONE kernel: plx_decode_partial whose last stage, instead of writing the
 * partial records, IS the exchange above -- the warp that holds the merged state of a (batch, head)
 * pushes it to every rank's inbox, waits (bounded, as above) for the peers' records and writes the merged
 * row of `out`.  Same inbox, same protocol and step count as plx_decode_exchange_merge (the two may be
 * mixed on one inbox), bit-identical result.  (No counterpart in the reference, which is single-GPU.)
 * Available for heads_q == heads_kv with 2 <= n_splits and the one-warp-per-split arrangement; otherwise
 * PLX_ERR_UNSUPPORTED is returned before anything is enqueued and the caller runs plx_decode_partial +
 * plx_decode_exchange_merge.  x->n_records, head_dim and dtype must match the problem. */
int plx_decode_partial_exchange(const plx_decode_problem *p, const plx_exchange *x, const void *q,
                                const void *r, const void *k, const void *v, void *out,
                                const int32_t *seqused_k, const int32_t *cache_start, void *workspace,
                                size_t workspace_bytes, plx_stream_t stream);

/* ------------------------------------------------------------------------- */
int plx_abi_version(void);
const char *plx_strerror(int status);
/* Every wait inside the pipelined (TMA / tcgen05) kernels and in the peer-memory exchange is
 * bounded; a kernel that gives up a wait records (site << 8) | 1 in a per-device error word and
 * returns, leaving the outputs of THAT launch undefined.  Kernels never read the word: an error
 * left behind does not change what later launches do.
 *   plx_device_error       SYNCHRONISES the current device, returns the word (first error since it
 *                          was cleared; 0 = none) and, if `clear` is non-zero, resets it.
 *   plx_device_error_peek  never synchronises: returns the copy of the report that the failing kernel
 *                          wrote to pinned host memory (0 until a report has arrived); `clear`
 *                          acknowledges it.  Cheap enough to call before every launch.
 * The first training or exchange call on a device allocates that host word (one small pinned
 * allocation per process): make it outside any stream capture. */
int plx_device_error(int32_t *value, int32_t clear);
int plx_device_error_peek(int32_t *value, int32_t clear);
/* Number of this library's kernels launched by the calling process so far. */
uint64_t plx_kernel_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* PLX_ABI_H */
