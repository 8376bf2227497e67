// extern "C" surface of libplx_sm100.so (declared in include/plx_abi.h):
// argument validation, kernel selection, launch accounting.
#include <atomic>

#include "plx_common.cuh"
#include "plx_decode.h"
#include "plx_launch.h"

namespace plx {

static std::atomic<uint64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// The kernels are built for sm_100a only; anything else must fail loudly, not fall back.
static int check_device() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return PLX_ERR_DEVICE;
    if (dev >= 0 && dev < 64) {
        int c = cached[dev].load(std::memory_order_relaxed);
        if (c != 0) return c > 0 ? PLX_OK : PLX_ERR_DEVICE;
    }
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return PLX_ERR_DEVICE;
    const bool ok = major == 10;
    if (dev >= 0 && dev < 64) cached[dev].store(ok ? 1 : -1, std::memory_order_relaxed);
    return ok ? PLX_OK : PLX_ERR_DEVICE;
}

static int check_train(const plx_train_problem *p) {
    if (!p) return PLX_ERR_BAD_ARG;
    if (p->batch <= 0 || p->heads_q <= 0 || p->heads_kv <= 0 || p->len_q <= 0 || p->len_k <= 0) return PLX_ERR_BAD_ARG;
    if (p->heads_q % p->heads_kv != 0) return PLX_ERR_BAD_ARG;
    if (p->window_left < -1) return PLX_ERR_BAD_ARG;
    if (p->dtype != PLX_BF16 && p->dtype != PLX_FP16) return PLX_ERR_UNSUPPORTED;
    if (p->head_dim != 64 && p->head_dim != 128) return PLX_ERR_UNSUPPORTED;
    if (p->cu_seqlens) {
        if (p->batch != 1 || p->n_seqs <= 0 || p->len_q != p->len_k) return PLX_ERR_BAD_ARG;
    }
    // 16-byte vector accesses: every stride must be a multiple of 8 elements
    const int64_t strides[] = {p->q_stride_b, p->q_stride_h, p->q_stride_t, p->kv_stride_b, p->kv_stride_h, p->kv_stride_t};
    for (int64_t s : strides)
        if (s < 0 || (s & 7) != 0) return PLX_ERR_BAD_ARG;
    if (static_cast<int64_t>(p->batch) * p->heads_q > 65535) return PLX_ERR_UNSUPPORTED;
    return PLX_OK;
}

static bool misaligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

static TrainArgs make_train_args(const plx_train_problem *p) {
    TrainArgs a{};
    a.cu = p->cu_seqlens;
    a.n_seqs = p->cu_seqlens ? p->n_seqs : 0;
    a.batch = p->batch;
    a.heads_q = p->heads_q;
    a.heads_kv = p->heads_kv;
    a.n_rep = p->heads_q / p->heads_kv;
    a.len_q = p->len_q;
    a.len_k = p->len_k;
    a.window = p->window_left;
    a.scale = p->qk_scale;
    a.c2 = p->qk_scale * kLog2e;
    a.q_sb = p->q_stride_b; a.q_sh = p->q_stride_h; a.q_st = p->q_stride_t;
    a.kv_sb = p->kv_stride_b; a.kv_sh = p->kv_stride_h; a.kv_st = p->kv_stride_t;
    a.st_sb = p->st_stride_b; a.st_sh = p->st_stride_h; a.st_st = p->st_stride_t;
    return a;
}

static size_t train_stat_rows(const plx_train_problem *p) {
    // one 64-row tile of slack: the dk/dv kernel fetches the statistics of whole 64-row tiles and the
    // last tile may reach past the last token
    return static_cast<size_t>(p->batch) * p->heads_q * p->len_q + 64;
}

static size_t train_ws_bytes(const plx_train_problem *p) {
    // per (batch, q head, token): an 8-float record plus a compact 4-float record (see bwd_stats_kernel)
    return train_stat_rows(p) * 12 * sizeof(float);
}

static int check_decode(const plx_decode_problem *p) {
    if (!p) return PLX_ERR_BAD_ARG;
    if (p->batch <= 0 || p->heads_q <= 0 || p->heads_kv <= 0 || p->cache_len <= 0 || p->n_splits <= 0 ||
        p->n_splits > PLX_DECODE_MAX_SPLITS)
        return PLX_ERR_BAD_ARG;
    if (p->heads_q % p->heads_kv != 0 || p->window_left < -1 || p->kv_offset < 0 || p->total_len < 0) return PLX_ERR_BAD_ARG;
    if (p->dtype != PLX_BF16 && p->dtype != PLX_FP16) return PLX_ERR_UNSUPPORTED;
    if (p->head_dim != 64 && p->head_dim != 128) return PLX_ERR_UNSUPPORTED;
    const int64_t strides[] = {p->kv_stride_b, p->kv_stride_t, p->kv_stride_h};
    for (int64_t s : strides)
        if (s < 0 || (s & 7) != 0) return PLX_ERR_BAD_ARG;
    if (p->heads_q > 65535 || p->batch > 65535) return PLX_ERR_UNSUPPORTED;
    if (p->page_table) {
        if (p->page_size < 1 || (p->page_size & (p->page_size - 1)) != 0 || p->pages_per_seq < 1) return PLX_ERR_BAD_ARG;
        if (static_cast<int64_t>(p->pages_per_seq) * p->page_size < p->cache_len) return PLX_ERR_BAD_ARG;
        if (p->kv_offset != 0) return PLX_ERR_UNSUPPORTED;   // a paged cache is not key-sharded
    }
    return PLX_OK;
}

static size_t decode_ws_bytes(const plx_decode_problem *p) {
    const size_t bh = static_cast<size_t>(p->batch) * p->heads_q;
    const size_t groups = PLX_DECODE_GROUPS(p->n_splits);
    return bh * (p->n_splits + groups) * PLX_DECODE_PART_FLOATS(p->head_dim) * sizeof(float) + bh * (1 + groups) * sizeof(int);
}

// the checks of a decode call that do not concern the workspace: problem, pointers, alignment, device
static int check_decode_args(const plx_decode_problem *p, const void *q, const void *r, const void *k, const void *v,
                             const void *out, const void *part) {
    int st = check_decode(p);
    if (st != PLX_OK) return st;
    if (!q || !r || !k || !v || (!out && !part)) return PLX_ERR_BAD_ARG;
    if (misaligned16(q) || misaligned16(r) || misaligned16(k) || misaligned16(v) || (out && misaligned16(out)))
        return PLX_ERR_BAD_ARG;
    return check_device();
}

// fills the kernel-side exchange block from the C struct; PLX_OK or the status to return
static int make_exchange_args(const plx_exchange *x, ExchangeArgs &e) {
    if (x->world < 1 || x->world > PLX_EXCHANGE_MAX_RANKS || x->rank < 0 || x->rank >= x->world || x->n_records <= 0)
        return PLX_ERR_BAD_ARG;
    if (x->head_dim != 64 && x->head_dim != 128) return PLX_ERR_UNSUPPORTED;
    for (int r = 0; r < x->world; ++r) {
        if (!x->inbox[r] || misaligned16(x->inbox[r])) return PLX_ERR_BAD_ARG;
        e.inbox[r] = static_cast<float *>(x->inbox[r]);
    }
    e.world = x->world; e.rank = x->rank; e.n_records = x->n_records;
    e.status = x->status;
    e.wait_ms = x->wait_ms ? x->wait_ms : PLX_EXCHANGE_DEFAULT_WAIT_MS;
    return PLX_OK;
}

static int run_decode(const plx_decode_problem *p, const void *q, const void *r, const void *k, const void *v, void *out,
                      float *part, const int32_t *seqused_k, const int32_t *cache_start, void *workspace,
                      size_t workspace_bytes, cudaStream_t stream, const plx_exchange *xch = nullptr) {
    int st = check_decode_args(p, q, r, k, v, out, part);
    if (st != PLX_OK) return st;
    if (p->n_splits > 1 && (!workspace || workspace_bytes < decode_ws_bytes(p) || misaligned16(workspace)))
        return PLX_ERR_WORKSPACE;
    DecodeArgs a{};
    a.q = q; a.r = r; a.k = k; a.v = v;
    a.out = part ? nullptr : out;
    a.part_out = part;
    a.seqused = seqused_k;
    a.cache_start = cache_start;
    const size_t bh = static_cast<size_t>(p->batch) * p->heads_q;
    // workspace: split records | group records | per-(batch, head) counters | group counters
    const size_t rec = PLX_DECODE_PART_FLOATS(p->head_dim), groups = PLX_DECODE_GROUPS(p->n_splits);
    a.n_groups = static_cast<int>(groups);
    a.ws_parts = static_cast<float *>(workspace);
    if (workspace) {
        a.ws_gparts = a.ws_parts + bh * p->n_splits * rec;
        a.ws_counters = reinterpret_cast<int *>(a.ws_gparts + bh * groups * rec);
        a.ws_gcounters = a.ws_counters + bh;
    }
    a.batch = p->batch; a.heads_q = p->heads_q; a.heads_kv = p->heads_kv; a.n_rep = p->heads_q / p->heads_kv;
    a.cache_len = p->cache_len; a.window = p->window_left; a.n_splits = p->n_splits;
    a.kv_offset = p->kv_offset;
    a.total_len = p->total_len > 0 ? p->total_len : p->cache_len;
    a.c2 = p->qk_scale * kLog2e;
    a.kv_sb = p->kv_stride_b; a.kv_st = p->kv_stride_t; a.kv_sh = p->kv_stride_h;
    if (xch) {
        if ((st = make_exchange_args(xch, a.xch)) != PLX_OK) return st;
        if (xch->n_records != p->batch * p->heads_q || xch->head_dim != p->head_dim || xch->dtype != p->dtype) return PLX_ERR_BAD_ARG;
        if (!decode_fused_exchange_supported(a)) return PLX_ERR_UNSUPPORTED;
        const ErrorWords ew = sm100_error_words();
        if (!ew.word) return PLX_ERR_LAUNCH;
        a.xch.err_word = ew.word;
        a.xch.err_mirror = ew.mirror;
    }
    a.page_table = p->page_table;
    if (p->page_table) {
        a.pages_per_seq = p->pages_per_seq;
        a.page_mask = p->page_size - 1;
        a.page_shift = 0;
        while ((1 << a.page_shift) < p->page_size) ++a.page_shift;
    }
    return launch_decode(a, p->dtype, p->head_dim, stream);
}

}  // namespace plx

using namespace plx;

extern "C" {

int plx_abi_version(void) { return PLX_ABI_VERSION; }

const char *plx_strerror(int status) {
    switch (status) {
        case PLX_OK: return "ok";
        case PLX_ERR_BAD_ARG: return "bad argument (null pointer, size, stride or alignment)";
        case PLX_ERR_UNSUPPORTED: return "unsupported dtype, head_dim or shape";
        case PLX_ERR_LAUNCH: return "CUDA kernel launch failed";
        case PLX_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case PLX_ERR_DEVICE: return "current CUDA device is not sm_100 (B200)";
        case PLX_ERR_STATIC_SCRATCH:
            return "problem needs more split-KV scratch than the built-in array of plx_decode_static; lower n_splits "
                   "or call plx_decode with a caller-owned workspace";
        default: return "unknown status";
    }
}

uint64_t plx_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int plx_device_error(int32_t *value, int32_t clear) {
    if (!value) return PLX_ERR_BAD_ARG;
    int v = 0;
    int st = sm100_error_word(&v, clear != 0);
    *value = v;
    return st;
}

int plx_device_error_peek(int32_t *value, int32_t clear) {
    if (!value) return PLX_ERR_BAD_ARG;
    int v = 0;
    int st = sm100_error_peek(&v, clear != 0);
    *value = v;
    return st;
}

int plx_train_workspace_bytes(const plx_train_problem *p, size_t *bytes) {
    int st = check_train(p);
    if (st != PLX_OK) return st;
    if (!bytes) return PLX_ERR_BAD_ARG;
    *bytes = train_ws_bytes(p);
    return PLX_OK;
}

int plx_train_fwd(const plx_train_problem *p, const void *q, const void *r, const void *k, const void *v, void *o,
                  void *barv, float *d1, float *bart, float *m, plx_stream_t stream) {
    int st = check_train(p);
    if (st != PLX_OK) return st;
    if (!q || !r || !k || !v || !o || !barv || !d1 || !bart || !m) return PLX_ERR_BAD_ARG;
    if (misaligned16(q) || misaligned16(r) || misaligned16(k) || misaligned16(v) || misaligned16(o) || misaligned16(barv))
        return PLX_ERR_BAD_ARG;
    if ((st = check_device()) != PLX_OK) return st;
    TrainArgs a = make_train_args(p);
    a.q = q; a.r = r; a.k = k; a.v = v; a.o = o; a.barv = barv; a.d1 = d1; a.bart = bart; a.m = m;
    if (train_fwd_sm100_supported(a, p->head_dim))
        return launch_train_fwd_sm100(a, p->dtype, p->head_dim, reinterpret_cast<cudaStream_t>(stream));
    return launch_train_fwd_mma(a, p->dtype, p->head_dim, reinterpret_cast<cudaStream_t>(stream));
}

int plx_train_bwd_stages(const plx_train_problem *p, int32_t stages, const void *q, const void *r, const void *k,
                         const void *v, const void *o, const void *barv, const float *d1, const float *bart,
                         const float *m, const void *grad_o, void *dq, void *dr, void *dk, void *dv, void *workspace,
                         size_t workspace_bytes, plx_stream_t stream) {
    int st = check_train(p);
    if (st != PLX_OK) return st;
    if (stages <= 0 || (stages & ~PLX_BWD_ALL) != 0) return PLX_ERR_BAD_ARG;
    if (!q || !r || !k || !v || !o || !barv || !d1 || !bart || !m || !grad_o || !dq || !dr || !dk || !dv)
        return PLX_ERR_BAD_ARG;
    const void *ptrs[] = {q, r, k, v, o, barv, grad_o, dq, dr, dk, dv};
    for (const void *x : ptrs)
        if (misaligned16(x)) return PLX_ERR_BAD_ARG;
    if (!workspace || workspace_bytes < train_ws_bytes(p) || misaligned16(workspace)) return PLX_ERR_WORKSPACE;
    if ((st = check_device()) != PLX_OK) return st;
    TrainArgs a = make_train_args(p);
    a.q = q; a.r = r; a.k = k; a.v = v; a.o_in = o; a.barv_in = barv; a.go = grad_o;
    a.d1 = const_cast<float *>(d1); a.bart = const_cast<float *>(bart); a.m = const_cast<float *>(m);
    a.dq = dq; a.dr = dr; a.dk = dk; a.dv = dv;
    a.bst = static_cast<float *>(workspace);
    a.cst = a.bst + train_stat_rows(p) * 8;
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
    const bool tc = train_bwd_sm100_supported(a, p->head_dim);
    for (int stage : {PLX_BWD_STATS, PLX_BWD_DQR, PLX_BWD_DKV}) {
        if (!(stages & stage)) continue;
        st = (tc && stage != PLX_BWD_STATS) ? launch_train_bwd_sm100(a, p->dtype, p->head_dim, stage, cs)
                                            : launch_train_bwd_mma(a, p->dtype, p->head_dim, stage, cs);
        if (st != PLX_OK) return st;
    }
    return PLX_OK;
}

int plx_train_bwd(const plx_train_problem *p, const void *q, const void *r, const void *k, const void *v, const void *o,
                  const void *barv, const float *d1, const float *bart, const float *m, const void *grad_o, void *dq,
                  void *dr, void *dk, void *dv, void *workspace, size_t workspace_bytes, plx_stream_t stream) {
    return plx_train_bwd_stages(p, PLX_BWD_ALL, q, r, k, v, o, barv, d1, bart, m, grad_o, dq, dr, dk, dv, workspace,
                                workspace_bytes, stream);
}

int plx_decode_choose_splits(int32_t batch, int32_t heads_q, int32_t n_keys, int32_t sm_count) {
    if (batch <= 0 || heads_q <= 0 || n_keys <= 0 || sm_count <= 0) return 1;
    // One warp per (batch, head, split).  Measured on B200: a launch is fastest when all its warps are
    // resident at once (16 per SM at this kernel's register count; one warp more starts a second wave
    // with a long tail, and more splits only add partial records to merge), unless that leaves more
    // than ~1024 keys to a warp, where several waves of smaller units balance better.  At least 32
    // keys per split.
    const int64_t bh = static_cast<int64_t>(batch) * heads_q;
    const int64_t resident = static_cast<int64_t>(sm_count) * 16;
    // Few (batch, head) pairs and not many keys: the launch is bound by latency.  Split groups (eight
    // splits per CTA, merged in shared memory): about 16 keys per warp, so that all of a warp's loads are
    // in flight at once, as long as every warp is resident; a multiple of 8, at most 256.
    if (bh <= PLX_DECODE_SPLIT_GROUP_MAX_BH && n_keys >= 128 && bh * n_keys <= (static_cast<int64_t>(1) << 19)) {
        if (n_keys <= 2048) {
            // at most eight CTAs per (batch, head): they form one thread-block cluster and merge through
            // distributed shared memory; 8, 16, 32 or 64 splits of at least 16 keys.  (Measured at B = 1,
            // H = 8: 4.8 / 6.1 us at 512 / 1024 keys.)
            int64_t g = 64;
            while (g > 8 && n_keys / g < 16) g /= 2;
            return static_cast<int>(g);
        }
        // Up to 6144 keys a cluster still wins where its CTAs are all resident at once and no warp walks
        // more than about 200 keys.  Measured (H = 8, cold K/V, us at 2560 / 3072 / 4096 / 6144 keys):
        // B = 1: 64 splits 7.9 / 7.9 / 9.4 / 11.8 against 9.6 / 10.2 / 11.0 / 12.2 for the rule below;
        // B = 4: 32 splits 12.4 / 13.8 / 16.5 / 21.7 against 14.5 / 16.2 / 19.2 / 24.1 (B = 3 alike);
        // B = 2, 6 and 8 are faster with the rule below.
        if (n_keys <= 6144) {
            if (bh <= 8) return 64;
            if (bh > 16 && bh <= 32) return 32;
        }
        int64_t g = (n_keys + 15) / 16;
        if (g > resident / bh) g = resident / bh;
        if (g > PLX_DECODE_MAX_SPLITS) g = PLX_DECODE_MAX_SPLITS;
        g -= g % 8;
        if (g >= 8) return static_cast<int>(g);
    }
    int64_t s = resident / bh;
    if (s < 1) s = 1;
    if (n_keys / s > 1024) s = (n_keys + 1023) / 1024;
    int64_t cap = n_keys / 32;
    if (cap < 1) cap = 1;
    if (s > cap) s = cap;
    if (s > PLX_DECODE_MAX_SPLITS) s = PLX_DECODE_MAX_SPLITS;
    return s < 1 ? 1 : static_cast<int>(s);
}

int plx_decode_choose_splits_gqa(int32_t batch, int32_t heads_q, int32_t heads_kv, int32_t n_keys, int32_t sm_count) {
    if (heads_kv <= 0 || heads_q <= heads_kv || heads_q % heads_kv != 0)
        return plx_decode_choose_splits(batch, heads_q, n_keys, sm_count);
    if (batch <= 0 || n_keys <= 0 || sm_count <= 0) return 1;
    // Grouped heads run one warp per (batch, kv head, 16-row head group, split), kDecodeGqaWarps
    // resident per SM (their K / V tiles fill the shared memory).  The warps of a launch run in waves of
    // that many: take the smallest split count whose last wave is at least 85 % full (or the fullest,
    // if none is), with at least 64 keys per split.
    const int64_t units = static_cast<int64_t>(batch) * heads_kv * ((heads_q / heads_kv + 15) / 16);
    const int64_t resident = static_cast<int64_t>(sm_count) * kDecodeGqaWarps;
    int64_t cap = n_keys / 64;
    if (cap < 1) cap = 1;
    if (cap > PLX_DECODE_MAX_SPLITS) cap = PLX_DECODE_MAX_SPLITS;
    int64_t best = 1;
    double best_fill = 0.0;
    for (int64_t s = 1; s <= cap; ++s) {
        const int64_t warps = units * s, waves = (warps + resident - 1) / resident;
        const double fill = static_cast<double>(warps) / static_cast<double>(waves * resident);
        if (fill > best_fill + 1e-9) {
            best_fill = fill;
            best = s;
        }
        if (fill >= 0.85) break;
    }
    return static_cast<int>(best);
}

int plx_decode_workspace_bytes(const plx_decode_problem *p, size_t *bytes) {
    int st = check_decode(p);
    if (st != PLX_OK) return st;
    if (!bytes) return PLX_ERR_BAD_ARG;
    *bytes = decode_ws_bytes(p);
    return PLX_OK;
}

// internal (not in plx_abi.h): lets plx_decode_static run plx_decode's checks before it enqueues its memset
int plx_decode_check_args(const plx_decode_problem *p, const void *q, const void *r, const void *k, const void *v,
                          const void *out) {
    if (!out) return PLX_ERR_BAD_ARG;
    return check_decode_args(p, q, r, k, v, out, nullptr);
}

int plx_decode(const plx_decode_problem *p, const void *q, const void *r, const void *k, const void *v, void *out,
               const int32_t *seqused_k, const int32_t *cache_start, void *workspace, size_t workspace_bytes,
               plx_stream_t stream) {
    if (!out) return PLX_ERR_BAD_ARG;
    return run_decode(p, q, r, k, v, out, nullptr, seqused_k, cache_start, workspace, workspace_bytes,
                      reinterpret_cast<cudaStream_t>(stream));
}

int plx_decode_partial(const plx_decode_problem *p, const void *q, const void *r, const void *k, const void *v,
                       float *part, const int32_t *seqused_k, const int32_t *cache_start, void *workspace,
                       size_t workspace_bytes, plx_stream_t stream) {
    if (!part) return PLX_ERR_BAD_ARG;
    return run_decode(p, q, r, k, v, nullptr, part, seqused_k, cache_start, workspace, workspace_bytes,
                      reinterpret_cast<cudaStream_t>(stream));
}

int plx_decode_merge(const float *parts, int32_t n_parts, int32_t n_records, int32_t head_dim, int32_t dtype, void *out,
                     plx_stream_t stream) {
    if (!parts || !out || n_parts <= 0 || n_records <= 0) return PLX_ERR_BAD_ARG;
    int st = check_device();
    if (st != PLX_OK) return st;
    return launch_decode_merge(parts, n_parts, n_records, head_dim, dtype, out, reinterpret_cast<cudaStream_t>(stream));
}

size_t plx_decode_exchange_bytes(int32_t world, int32_t n_records, int32_t head_dim) {
    if (world <= 0 || n_records <= 0 || (head_dim != 64 && head_dim != 128)) return 0;
    const size_t slots = static_cast<size_t>(2) * world * n_records;   // two parities
    return slots * PLX_DECODE_PART_FLOATS(head_dim) * sizeof(float) + slots * sizeof(uint32_t) +
           static_cast<size_t>(n_records) * sizeof(uint32_t);   // records, stamps, step counters
}

int plx_decode_partial_exchange(const plx_decode_problem *p, const plx_exchange *x, const void *q, const void *r,
                                const void *k, const void *v, void *out, const int32_t *seqused_k,
                                const int32_t *cache_start, void *workspace, size_t workspace_bytes, plx_stream_t stream) {
    if (!x || !out) return PLX_ERR_BAD_ARG;
    return run_decode(p, q, r, k, v, out, nullptr, seqused_k, cache_start, workspace, workspace_bytes,
                      reinterpret_cast<cudaStream_t>(stream), x);
}

int plx_decode_exchange_merge(const plx_exchange *x, const float *part, void *out, plx_stream_t stream) {
    if (!x || !part || !out) return PLX_ERR_BAD_ARG;
    if (misaligned16(part) || misaligned16(out)) return PLX_ERR_BAD_ARG;
    ExchangeArgs e{};
    int st = make_exchange_args(x, e);
    if (st != PLX_OK) return st;
    if ((st = check_device()) != PLX_OK) return st;
    const ErrorWords err = sm100_error_words();
    if (!err.word) return PLX_ERR_LAUNCH;
    return launch_decode_exchange_merge(e, part, x->head_dim, x->dtype, out, err, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
