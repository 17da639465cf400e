// Host-side launch helpers shared by the operator entry points and the decoder.
#pragma once
#include <cuda.h>

#include "attention.cuh"
#include "gemv.cuh"
#include "gemv_stream.cuh"
#include "gemv_pair.cuh"
#include "gemv_ksplit.cuh"
#include "gemv_mma.cuh"
#include "gemv_q5k.cuh"
#include "moe.cuh"
#include "prefill_gemm.cuh"
#include "q8k.cuh"
#include "state.hpp"

namespace rnb {

// Programmatic dependent launch (off with RNB_B200_PDL=0): kernels overlap their weight
// prefetch and set-up with the tail of the previous kernel.  EVERY kernel launched through
// launch_k must execute pdl_wait() before it touches memory another kernel wrote: a kernel
// that skips it neither waits for its predecessor nor orders its successor behind it.
bool use_pdl();

// Kernels launched by this library so far (callers take differences).
inline uint64_t &launch_count() {
    static uint64_t n = 0;
    return n;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    if (use_pdl()) {
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e == cudaSuccess) launch_count()++;
    return e;
}

// The same launch as one thread-block cluster per grid column: cluster dimensions (1, cluster_y, 1).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, unsigned cluster_y, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = cluster_y;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (e == cudaSuccess) launch_count()++;
    return e;
}

constexpr size_t GEMV_SMEM_LIMIT = 200 * 1024;

// Rows per tile: tiles are whole rows, their byte size must be a multiple of 16 for the bulk
// copy, about 16 KB each, and there should be a few tiles per SM so the tail is short.
inline int pick_rows_per_tile(int type, size_t rows, size_t cols, int n_parts, int sm_count) {
    const size_t rb = row_bytes_of(type, cols);
    if (rb == 0) return 1;
    size_t unit = 1;
    while ((unit * rb) % 16 != 0) unit *= 2;  // rb is even for every format: unit <= 8
    size_t r = (16384 / rb) / unit * unit;
    if (r < unit) r = unit;
    while (r > unit && (rows + r - 1) / r < (size_t)(4 * sm_count) && r * rb > 4096) r -= unit;
    while (r > unit && (size_t)n_parts * (r * rb + 32) > GEMV_SMEM_LIMIT) r -= unit;
    if (r > rows) r = (rows + unit - 1) / unit * unit;
    return (int)r;
}
inline uint32_t gemv_part_stride(int type, size_t cols, int rows_per_tile) {
    return (uint32_t)(((size_t)rows_per_tile * row_bytes_of(type, cols) + 15) & ~(size_t)15) + 16;
}

int gemv_kernel_setup();  // raises the dynamic shared memory limit once
size_t gemv_smem_max();    // dynamic shared memory a matvec launch may ask for

// Streaming (batch-1) kernel geometry: rows per CTA (0 = choose per launch), super-blocks per
// stage and pipeline depth; overridable by RNB_B200_GEMV_ROWS / _CHUNK / _STAGES for tuning.
struct GemvTuning {
    int rows, chunk_blocks, stages;
};
const GemvTuning &gemv_tuning();

inline bool gemv_use_stream(int type, int seq, size_t cols) {
    return seq <= 1 && cols % 256 == 0 && (type == TYPE_Q4_K || type == TYPE_Q6_K);
}
// Rows per CTA for the streaming kernel (4 per warp): 8 when that still leaves two CTAs per SM
// (measured inside a decode step: 4096-row matrices are 1 % faster with 8), else 4.
inline int gs_pick_rows(size_t total_rows, int sm_count) {
    const int forced = gemv_tuning().rows;
    if (forced == 4 || forced == 8 || forced == 16) return forced;
    return (total_rows + 7) / 8 >= (size_t)(2 * sm_count) ? 8 : 4;
}

inline int launch_gemv_stream_rows(cudaStream_t s, const GemvJob *jobs_host, const GemvJob *jobs_dev, int n_jobs,
                                   size_t cols, int *dev_error, int dynamic_table, bool by_value) {
    const GemvTuning &tu = gemv_tuning();
    const int R = jobs_host[0].rows_per_tile;
    int tiles = 0, max_parts = 1;
    uint32_t blk = 0;
    for (int i = 0; i < n_jobs; i++) {
        const GemvJob &j = jobs_host[i];
        if (j.rows_per_tile != R || (R != 4 && R != 8 && R != 16) || !gemv_use_stream(j.type, j.seq, cols))
            return fail(RNB_B200_VALIDATION_FAILED, "matvec jobs of one launch must share a valid rows-per-CTA and be K-quants");
        tiles = j.tile0 + (j.rows + R - 1) / R;
        if (j.n_parts > max_parts) max_parts = j.n_parts;
        const uint32_t bb = j.type == TYPE_Q4_K ? Q4K_BYTES : Q6K_BYTES;
        if (bb > blk) blk = bb;
    }
    const int nb = (int)(cols / 256);
    GsParams P;
    P.cols = (int)cols;
    P.rows_per_cta = R;
    P.chunk_blocks = tu.chunk_blocks < nb ? tu.chunk_blocks : nb;
    const int n_items = (nb + P.chunk_blocks - 1) / P.chunk_blocks * max_parts;
    P.n_stages = n_items < tu.stages ? n_items : tu.stages;
    P.row_stride = (((uint32_t)P.chunk_blocks * blk + 15u) & ~15u) + 16u;  // rows stay 16-byte aligned
    P.act_off = (uint32_t)R * P.row_stride;
    P.slot_bytes = P.act_off + (uint32_t)P.chunk_blocks * 288u;
    P.dynamic_table = dynamic_table;
    size_t smem = (size_t)P.n_stages * P.slot_bytes;
    while (smem > gemv_smem_max() && P.n_stages > 1) smem = (size_t)(--P.n_stages) * P.slot_bytes;
    if (smem > gemv_smem_max()) return fail(RNB_B200_VALIDATION_FAILED, "matvec stage too large: %zu bytes", smem);
    if ((by_value || !dynamic_table) && n_jobs <= GS_PACK) {
        GemvJobPack pack;
        memset(&pack, 0, sizeof(pack));
        for (int i = 0; i < n_jobs; i++) pack.j[i] = jobs_host[i];
        RNB_CU(launch_k(gemv_stream_kernel_1, dim3(tiles), dim3(R * 8), smem, s, pack, n_jobs, P, dev_error));
    } else {
        RNB_CU(launch_k(gemv_stream_kernel, dim3(tiles), dim3(R * 8), smem, s, jobs_dev, n_jobs, P, dev_error));
    }
    return RNB_B200_OK;
}

// Tuning of the two-threads-per-row kernel: RNB_B200_PAIR=0 turns it off, _MIN_ROWS / _CHUNK /
// _STAGES override when it is used and its pipeline shape.
struct PairTuning {
    int enabled, min_rows, chunk, stages;
};
inline const PairTuning &pair_tuning() {
    static const PairTuning t = [] {
        auto env_int = [](const char *name, int dflt, int lo, int hi) {
            const char *e = getenv(name);
            if (!e || !*e) return dflt;
            const int x = atoi(e);
            return x < lo ? lo : (x > hi ? hi : x);
        };
        PairTuning v;
        v.enabled = env_int("RNB_B200_PAIR", 1, 0, 1);
        v.min_rows = env_int("RNB_B200_PAIR_MIN_ROWS", 16384, 0, 1 << 30);
        v.chunk = env_int("RNB_B200_PAIR_CHUNK", 2, 1, GP_MAX_CHUNK);
        v.stages = env_int("RNB_B200_PAIR_STAGES", 3, 1, GP_MAX_STAGES);
        return v;
    }();
    return t;
}
// K-split kernel: single static Q6_K job with long rows and few of them - the row-sharded
// ffn_down slices of a multi-GPU run (1024 x 28672 on 8 GPUs); with 4096 rows it is faster alone
// but not inside a decode step.  RNB_B200_KSPLIT=0 turns it off, _MIN_COLS / _MAX_ROWS move the limits.
struct KsplitTuning {
    int enabled, min_cols, max_rows, stages;
};
inline const KsplitTuning &ksplit_tuning() {
    static const KsplitTuning t = [] {
        auto env_int = [](const char *name, int dflt) {
            const char *e = getenv(name);
            return (e && *e) ? atoi(e) : dflt;
        };
        KsplitTuning v;
        v.enabled = env_int("RNB_B200_KSPLIT", 1);
        v.min_cols = env_int("RNB_B200_KSPLIT_MIN_COLS", 8192);
        v.max_rows = env_int("RNB_B200_KSPLIT_MAX_ROWS", 2048);
        v.stages = env_int("RNB_B200_KSPLIT_STAGES", 3);
        if (v.stages < 1) v.stages = 1;
        if (v.stages > GK_MAX_STAGES) v.stages = GK_MAX_STAGES;
        return v;
    }();
    return t;
}
// Integer-MMA kernel (gemv_mma.cuh): every batch-1 Q4_K / Q6_K launch whose operands are 16-byte
// aligned (Q6_K rows additionally need a multiple of 8 super-blocks, so that every stage starts
// on a 16-byte boundary).  RNB_B200_MMA=0 turns it off, _MMA_STAGES / _MMA_CTAS set the ring depth
// and the resident CTAs per SM the persistent grid is sized for.
// Descriptor of a weight matrix for the integer-MMA matvec's tiled copies: [rows][row_bytes / 8] 8-byte
// words, boxes of 16 rows x box_bytes / 8 words, no swizzle, zeros outside the matrix.
int encode_weight_map(GmTensorMap *out, const uint8_t *w, size_t rows, size_t row_bytes, uint32_t box_bytes);
struct MmaTuning {
    int enabled, stages, ctas_per_sm, chunk16, tmap;
};
inline const MmaTuning &mma_tuning() {
    static const MmaTuning t = [] {
        auto env_int = [](const char *name, int dflt, int lo, int hi) {
            const char *e = getenv(name);
            if (!e || !*e) return dflt;
            const int x = atoi(e);
            return x < lo ? lo : (x > hi ? hi : x);
        };
        MmaTuning v;
        v.enabled = env_int("RNB_B200_MMA", 1, 0, 1);
        v.stages = env_int("RNB_B200_MMA_STAGES", 3, 1, GM_MAX_STAGES);
        v.ctas_per_sm = env_int("RNB_B200_MMA_CTAS", 0, 0, 8);
        v.chunk16 = env_int("RNB_B200_MMA_CHUNK16", 1, 0, 1);
        v.tmap = env_int("RNB_B200_MMA_TMAP", 1, 0, 1);
        return v;
    }();
    return t;
}
// Returns 1 when the launch was taken, 0 when the jobs do not qualify, < 0 on error.
inline int try_launch_gemv_mma(cudaStream_t s, const GemvJob *jobs_host, const GemvJob *jobs_dev, int n_jobs, size_t cols, int *dev_error,
                               int dynamic_table, bool by_value, const GpTail *tail, bool *tail_done) {
    const MmaTuning &mt = mma_tuning();
    if (!mt.enabled || cols % 256 != 0 || n_jobs < 1) return 0;
    const int nb = (int)(cols / 256);
    bool any_q6 = false;
    int tiles = 0;
    for (int i = 0; i < n_jobs; i++) {
        const GemvJob &j = jobs_host[i];
        if ((j.type != TYPE_Q4_K && j.type != TYPE_Q6_K) || j.seq > 1 || j.n_parts < 1 || j.n_parts > GEMV_MAX_PARTS || j.rows < 1) return 0;
        if (j.type == TYPE_Q6_K) {
            any_q6 = true;
            if (nb % GM_CHUNK != 0) return 0;
        }
        for (int p = 0; p < j.n_parts; p++) {
            // device-written tables carry the weight pointers only on the device: expert slices are whole rows
            // of 16-byte multiples behind an allocation boundary
            if (!dynamic_table && (((uintptr_t)j.parts[p].w) & 15u)) return 0;
            if (((uintptr_t)j.parts[p].x) & 15u) return 0;
        }
        tiles += (j.rows + GM_ROWS - 1) / GM_ROWS;
    }
    // Row-rich Q4_K launches with short rows (gate + up: 28672 x 4096) stay on the two-threads-per-row kernel,
    // which measured faster there (14.9 us against 25 us): too few tiles per persistent CTA for this kernel's
    // pipeline to reach steady state.  RNB_B200_MMA_ALL=1 sends them here as well.
    static const bool all_shapes = [] {
        const char *e = getenv("RNB_B200_MMA_ALL");
        return e && *e == '1';
    }();
    if (!all_shapes && !any_q6 && !dynamic_table && tiles * GM_ROWS >= pair_tuning().min_rows && pair_tuning().enabled && nb <= 32) return 0;
    GmParams P;
    P.cols = (int)cols;
    P.dynamic_table = dynamic_table;
    P.n_tiles = tiles;
    // Stage geometry: 8 super-blocks per row when a Q6_K matrix is in the launch (8 x 210 bytes is its shortest
    // 16-byte multiple), else 16 (half as many copies to issue per byte); rows padded to an odd number of
    // 16-byte units so that ldmatrix reads eight rows without bank conflicts.
    // With tiled-copy descriptors (static single-part jobs that travel by value) a stage costs one copy
    // instruction whatever its width: 8 blocks per stage, each type at its own row pitch, a deeper ring.
    bool all_q6 = true, single_part = true;
    for (int i = 0; i < n_jobs; i++) {
        all_q6 = all_q6 && jobs_host[i].type == TYPE_Q6_K;
        single_part = single_part && jobs_host[i].n_parts == 1;
    }
    const bool by_val = (by_value || !dynamic_table) && n_jobs <= GS_PACK;
    P.use_tmap = (mt.tmap && by_val && !dynamic_table && single_part) ? 1 : 0;
    if (P.use_tmap) {
        P.chunk = GM_CHUNK;
        P.row_stride = 1168u;
        P.row_stride6 = any_q6 ? 1712u : 1168u;   // no Q6_K job: the slot is sized for Q4_K rows alone
        P.act_off = (uint32_t)GM_ROWS * P.row_stride6;
    } else {
        P.chunk = (any_q6 || nb < 2 * GM_CHUNK || mt.chunk16 == 0) ? GM_CHUNK : 2 * GM_CHUNK;
        P.row_stride = any_q6 ? 1712u : (P.chunk == GM_CHUNK ? 1168u : 2320u);
        P.row_stride6 = P.row_stride;
        P.act_off = (uint32_t)GM_ROWS * P.row_stride;
    }
    (void)all_q6;
    P.slot_bytes = (P.act_off + (uint32_t)P.chunk * GM_ACT_BLOCK_BYTES + 127u) & ~127u;
    int n_items = 0;
    for (int i = 0; i < n_jobs; i++) n_items = std::max(n_items, jobs_host[i].n_parts * ((nb + P.chunk - 1) / P.chunk));
    P.n_stages = P.use_tmap ? std::max(mt.stages, 4) : mt.stages;
    while (P.n_stages > 1 && gm_smem_bytes(P.n_stages, P.slot_bytes) > gemv_smem_max()) P.n_stages--;
    // two CTAs per SM (the kernels' register budget) matter more than a deeper ring
    const size_t per_cta_for_two = ((size_t)228 * 1024 - 2 * 1024) / 2;
    if (mt.ctas_per_sm != 1)
        while (P.n_stages > 2 && gm_smem_bytes(P.n_stages, P.slot_bytes) > per_cta_for_two) P.n_stages--;
    const size_t smem = gm_smem_bytes(P.n_stages, P.slot_bytes);
    if (smem > gemv_smem_max()) return 0;
    const int sm = state().sm_count > 0 ? state().sm_count : 148;
    int per_sm = mt.ctas_per_sm;
    if (per_sm == 0) {
        per_sm = (int)((size_t)227 * 1024 / (smem + 1024));
        if (per_sm > GM_MIN_CTAS) per_sm = GM_MIN_CTAS;   // the kernels' register budget is set for this many
        if (per_sm < 1) per_sm = 1;
    }
    const int grid = std::min(tiles, per_sm * sm);
    GpTail t;
    memset(&t, 0, sizeof(t));
    if (tail && tail->kind == 1 && !dynamic_table && n_jobs == 2 && jobs_host[0].rows == jobs_host[1].rows && jobs_host[0].rows % 256 == 0 &&
        jobs_host[0].rows == tail->n) {
        t = *tail;
        if (tail_done) *tail_done = true;
    }
    // kind 2: the rows of a single plain job also go to every peer's gathered buffer (sharded decode)
    if (tail && tail->kind == 2 && !dynamic_table && n_jobs == 1 && jobs_host[0].epi == GEMV_EPI_NONE && n_jobs <= GS_PACK) {
        t = *tail;
        t.peer.n_arrive = grid;
        if (tail_done) *tail_done = true;
    }
    if ((by_value || !dynamic_table) && n_jobs <= GS_PACK) {
        GemvJobPack pack;
        memset(&pack, 0, sizeof(pack));
        for (int i = 0; i < n_jobs; i++) pack.j[i] = jobs_host[i];
        GmTmaps tm;
        memset(&tm, 0, sizeof(tm));
        if (P.use_tmap)
            for (int i = 0; i < n_jobs; i++) {
                const GemvJob &j = jobs_host[i];
                const int rc = encode_weight_map(&tm.m[i], j.parts[0].w, (size_t)j.rows, row_bytes_of(j.type, cols), j.type == TYPE_Q4_K ? P.row_stride : P.row_stride6);
                if (rc != RNB_B200_OK) return -rc;
            }
        const cudaError_t e = t.kind == 2 ? launch_k(gemv_mma_kernel_1_peer, dim3(grid), dim3(GM_THREADS), smem, s, pack, n_jobs, P, dev_error, t, tm)
                                          : launch_k(gemv_mma_kernel_1, dim3(grid), dim3(GM_THREADS), smem, s, pack, n_jobs, P, dev_error, t, tm);
        if (e != cudaSuccess) return -fail_cuda(e, "gemv_mma_kernel launch");
    } else {
        if (t.kind) return -fail(RNB_B200_VALIDATION_FAILED, "matvec tail needs a by-value job table");
        const cudaError_t e = launch_k(gemv_mma_kernel, dim3(grid), dim3(GM_THREADS), smem, s, jobs_dev, n_jobs, P, dev_error);
        if (e != cudaSuccess) return -fail_cuda(e, "gemv_mma_kernel launch");
    }
    return 1;
}
// Row-rich, all-Q4_K, single-part, 16-byte aligned static tables go to the two-threads-per-row
// kernel; everything else to the eight-threads-per-row kernel.
inline int launch_gemv_pair_dyn(cudaStream_t s, const GemvJob *jobs_host, int n_jobs, size_t cols, int *dev_error, const GpTail *tail, bool *tail_done);
inline int launch_gemv_stream(cudaStream_t s, const GemvJob *jobs_host, const GemvJob *jobs_dev, int n_jobs,
                              size_t cols, int *dev_error, int dynamic_table, bool by_value, const GpTail *tail = nullptr,
                              bool *tail_done = nullptr) {
    if (n_jobs >= 1 && jobs_host[0].dyn_ids) return launch_gemv_pair_dyn(s, jobs_host, n_jobs, cols, dev_error, tail, tail_done);
    {
        const int took = try_launch_gemv_mma(s, jobs_host, jobs_dev, n_jobs, cols, dev_error, dynamic_table, by_value, tail, tail_done);
        if (took < 0) return -took;
        if (took) return RNB_B200_OK;
    }
    const KsplitTuning &kt = ksplit_tuning();
    if (kt.enabled && !dynamic_table && n_jobs == 1 && jobs_host[0].type == TYPE_Q6_K && jobs_host[0].n_parts == 1 && jobs_host[0].seq <= 1 && jobs_host[0].epi == GEMV_EPI_NONE &&
        cols % (256 * GK_CHUNK) == 0 && (int)cols >= kt.min_cols && jobs_host[0].rows <= kt.max_rows &&
        ((((uintptr_t)jobs_host[0].parts[0].w | (uintptr_t)jobs_host[0].parts[0].x) & 15u) == 0) && gk_smem(kt.stages) <= gemv_smem_max()) {
        const int tiles = (jobs_host[0].rows + GK_ROWS - 1) / GK_ROWS;
        const int n_chunks = (int)(cols / (256 * GK_CHUNK));
        const int S = kt.stages < n_chunks ? kt.stages : n_chunks;
        RNB_CU(launch_k(gemv_ksplit_q6k_kernel, dim3(tiles), dim3(GK_THREADS), (size_t)gk_smem(S), s, jobs_host[0], (int)cols, S, dev_error));
        return RNB_B200_OK;
    }
    const PairTuning &pt = pair_tuning();
    bool pair = pt.enabled && !dynamic_table && n_jobs <= GS_PACK && cols % 256 == 0;
    size_t total_rows = 0;
    for (int i = 0; i < n_jobs && pair; i++) {
        const GemvJob &j = jobs_host[i];
        pair = j.type == TYPE_Q4_K && j.n_parts == 1 && j.seq <= 1 && j.epi == GEMV_EPI_NONE && ((((uintptr_t)j.parts[0].w | (uintptr_t)j.parts[0].x) & 15u) == 0);
        total_rows += (size_t)j.rows;
    }
    if (!pair || total_rows < (size_t)pt.min_rows)
        return launch_gemv_stream_rows(s, jobs_host, jobs_dev, n_jobs, cols, dev_error, dynamic_table, by_value);
    GemvJobPack pack;
    memset(&pack, 0, sizeof(pack));
    int tiles = 0;
    for (int i = 0; i < n_jobs; i++) {
        pack.j[i] = jobs_host[i];
        pack.j[i].rows_per_tile = GP_ROWS;
        pack.j[i].tile0 = tiles;
        tiles += (jobs_host[i].rows + GP_ROWS - 1) / GP_ROWS;
    }
    const int nb = (int)(cols / 256);
    GpParams P;
    P.cols = (int)cols;
    P.chunk = pt.chunk < nb ? pt.chunk : nb;
    const int n_chunks = (nb + P.chunk - 1) / P.chunk;
    P.n_stages = n_chunks < pt.stages ? n_chunks : pt.stages;
    P.row_stride = (uint32_t)P.chunk * Q4K_BYTES;
    while ((P.row_stride & 127u) != 32u && (P.row_stride & 127u) != 96u) P.row_stride += 16u;
    P.rows_per_tile = GP_ROWS;
    P.act_off = ((uint32_t)GP_ROWS * P.row_stride + 127u) & ~127u;
    P.slot_bytes = (P.act_off + (uint32_t)P.chunk * 288u + 32u + 127u) & ~127u;
    const size_t smem = (size_t)P.n_stages * P.slot_bytes;
    if (smem > gemv_smem_max()) return launch_gemv_stream_rows(s, jobs_host, jobs_dev, n_jobs, cols, dev_error, dynamic_table, by_value);
    GpTail t;
    memset(&t, 0, sizeof(t));
    // the tail needs whole 256-row blocks of both vectors in this launch
    if (tail && tail->kind == 1 && n_jobs == 2 && jobs_host[0].rows == jobs_host[1].rows && jobs_host[0].rows % 256 == 0 && jobs_host[0].rows == tail->n) {
        t = *tail;
        if (tail_done) *tail_done = true;
    }
    RNB_CU(launch_k(gemv_pair_q4k_kernel, dim3(tiles), dim3(32), smem, s, pack, n_jobs, P, dev_error, t));
    return RNB_B200_OK;
}

// Rows per one-warp CTA of the expert-gathered matvec (RNB_B200_MOE_ROWS = 4, 8 or 16; the tail counters of the
// callers are sized for 4).  Measured on the 48-layer MoE shape: 16 rows 2.996 ms per token, 8 rows 3.033, 4 rows 3.124 -
// more, shorter warps do not pay although each warp is latency-bound.
inline int moe_rows_per_tile() {
    static const int v = [] {
        const char *e = getenv("RNB_B200_MOE_ROWS");
        const int x = (e && *e) ? atoi(e) : 16;
        return (x == 4 || x == 8 || x == 16) ? x : 16;
    }();
    return v;
}
// Expert-gathered jobs (GemvJob::dyn_ids): static tables by value, the two-threads-per-row kernel's expert form.
// Tunables: RNB_B200_MOE_CHUNK (super-blocks per stage, default min(4, row)), RNB_B200_MOE_STAGES (default 3).
inline int launch_gemv_pair_dyn(cudaStream_t s, const GemvJob *jobs_host, int n_jobs, size_t cols, int *dev_error, const GpTail *tail, bool *tail_done) {
    if (n_jobs > GS_PACK || cols % 256 != 0) return fail(RNB_B200_VALIDATION_FAILED, "expert-gathered matvec: at most %d jobs, cols a multiple of 256", GS_PACK);
    GemvJobPack pack;
    memset(&pack, 0, sizeof(pack));
    int tiles = 0;
    const int rpt = moe_rows_per_tile();
    for (int i = 0; i < n_jobs; i++) {
        const GemvJob &j = jobs_host[i];
        if (!j.dyn_ids || j.type != TYPE_Q4_K || j.n_parts != 1 || j.seq > 1 || j.epi != GEMV_EPI_NONE || j.dyn_rows < rpt || j.dyn_rows % rpt || j.rows % j.dyn_rows ||
            ((((uintptr_t)j.parts[0].w | (uintptr_t)j.parts[0].x) | (uintptr_t)j.dyn_x_stride) & 15u))
            return fail(RNB_B200_VALIDATION_FAILED, "expert-gathered matvec: Q4_K, one part, 16-byte aligned operands, whole tiles per expert");
        pack.j[i] = j;
        pack.j[i].rows_per_tile = rpt;
        pack.j[i].tile0 = tiles;
        tiles += j.rows / rpt;
    }
    static const int env_chunk = [] {
        const char *e = getenv("RNB_B200_MOE_CHUNK");
        return (e && *e) ? atoi(e) : 4;
    }();
    static const int env_stages = [] {
        const char *e = getenv("RNB_B200_MOE_STAGES");
        return (e && *e) ? atoi(e) : 3;
    }();
    const int nb = (int)(cols / 256);
    GpParams P;
    P.cols = (int)cols;
    P.chunk = std::max(1, std::min(std::min(env_chunk, GP_MAX_CHUNK), nb));
    const int n_chunks = (nb + P.chunk - 1) / P.chunk;
    P.n_stages = std::max(1, std::min(std::min(env_stages, GP_MAX_STAGES), n_chunks));
    P.row_stride = (uint32_t)P.chunk * Q4K_BYTES;
    while ((P.row_stride & 127u) != 32u && (P.row_stride & 127u) != 96u) P.row_stride += 16u;
    P.rows_per_tile = rpt;
    P.act_off = ((uint32_t)rpt * P.row_stride + 127u) & ~127u;
    P.slot_bytes = (P.act_off + (uint32_t)P.chunk * 288u + 32u + 127u) & ~127u;
    const size_t smem = (size_t)P.n_stages * P.slot_bytes;
    if (smem > gemv_smem_max()) return fail(RNB_B200_VALIDATION_FAILED, "expert-gathered matvec: stage ring of %zu bytes", smem);
    GpTail t;
    memset(&t, 0, sizeof(t));
    if (tail && tail->kind == 1 && n_jobs == 2 && jobs_host[0].rows == jobs_host[1].rows && jobs_host[0].rows % 256 == 0 && jobs_host[0].rows == tail->n &&
        (tail->vec_n == 0 || (tail->vec_n % 256 == 0 && tail->n % tail->vec_n == 0))) {
        t = *tail;
        if (tail_done) *tail_done = true;
    }
    if (tail && tail->kind == 3 && n_jobs == 1 && tail->n == jobs_host[0].dyn_rows && tail->sum_k * tail->n == jobs_host[0].rows && tail->gate == jobs_host[0].y) {
        t = *tail;
        if (tail_done) *tail_done = true;
    }
    RNB_CU(launch_k(gemv_pair_q4k_dyn_kernel, dim3(tiles), dim3(32), smem, s, pack, n_jobs, P, dev_error, t));
    return RNB_B200_OK;
}

// Launch a table of jobs that all share `cols`.  jobs_host is used to size the launch;
// jobs_dev is the same table in device memory.
inline int launch_gemv_jobs(cudaStream_t s, const GemvJob *jobs_host, const GemvJob *jobs_dev,
                            int n_jobs, size_t cols, int *dev_error, int dynamic_table = 0, const GpTail *tail = nullptr,
                            bool *tail_done = nullptr) {
    RNB_TRY(gemv_kernel_setup());
    if (gemv_use_stream(jobs_host[0].type, jobs_host[0].seq, cols))
        return launch_gemv_stream(s, jobs_host, jobs_dev, n_jobs, cols, dev_error, dynamic_table, false, tail, tail_done);
    int tiles = 0, max_parts = 1;
    uint32_t stride = 0;
    for (int i = 0; i < n_jobs; i++) {
        const GemvJob &j = jobs_host[i];
        tiles = j.tile0 + (j.rows + j.rows_per_tile - 1) / j.rows_per_tile;
        if (j.n_parts > max_parts) max_parts = j.n_parts;
        uint32_t st = gemv_part_stride(j.type, cols, j.rows_per_tile);
        if (st > stride) stride = st;
    }
    const size_t smem = (size_t)stride * max_parts;
    if (smem > gemv_smem_max()) return fail(RNB_B200_VALIDATION_FAILED, "matvec tile too large: %zu bytes", smem);
    RNB_CU(launch_k(gemv_tile_kernel, dim3(tiles), dim3(GEMV_THREADS), smem, s, jobs_dev, n_jobs,
                    (int)cols, stride, dev_error, dynamic_table));
    return RNB_B200_OK;
}
inline int launch_gemv_one(cudaStream_t s, const GemvJob &job, size_t cols, int *dev_error) {
    RNB_TRY(gemv_kernel_setup());
    if (gemv_use_stream(job.type, job.seq, cols)) return launch_gemv_stream(s, &job, nullptr, 1, cols, dev_error, 0, true);
    const int tiles = (job.rows + job.rows_per_tile - 1) / job.rows_per_tile;
    const uint32_t stride = gemv_part_stride(job.type, cols, job.rows_per_tile);
    const size_t smem = (size_t)stride * job.n_parts;
    if (smem > gemv_smem_max()) return fail(RNB_B200_VALIDATION_FAILED, "matvec tile too large: %zu bytes", smem);
    RNB_CU(launch_k(gemv_tile_kernel_1, dim3(tiles), dim3(GEMV_THREADS), smem, s, job, (int)cols,
                    stride, dev_error));
    return RNB_B200_OK;
}
// rows_per_tile: 0 = automatic.  Batch-1 K-quant jobs run on the streaming kernel (4, 8 or 16
// rows per CTA); batched and Q8_0 jobs keep whole-row tiles in shared memory.
inline GemvJob make_job(int type, const uint8_t *w, const void *x, float *y, const float *residual,
                        size_t rows, size_t cols, int rows_per_tile, int sm_count, int seq = 1,
                        size_t x_stride = 0, int n_parts = 1) {
    GemvJob j;
    memset(&j, 0, sizeof(j));
    j.y = y;
    j.residual = residual;
    j.rows = (int)rows;
    j.type = type;
    j.n_parts = n_parts;
    j.tile0 = 0;
    if (gemv_use_stream(type, seq, cols))
        j.rows_per_tile = (rows_per_tile == 4 || rows_per_tile == 8 || rows_per_tile == 16) ? rows_per_tile : gs_pick_rows(rows, sm_count);
    else
        j.rows_per_tile = rows_per_tile > 0 ? rows_per_tile : pick_rows_per_tile(type, rows, cols, n_parts, sm_count);
    j.seq = seq;
    j.x_stride = x_stride;
    j.parts[0].w = w;
    j.parts[0].x = reinterpret_cast<const uint8_t *>(x);
    j.parts[0].scale = nullptr;
    return j;
}
// Jobs that go out in one launch: pick the common rows-per-CTA (streaming kernel) and lay the
// jobs' tiles end to end.
inline void gemv_finalize_group(GemvJob *jobs, int n, size_t cols, int sm_count) {
    bool stream = true;
    size_t total_rows = 0;
    for (int i = 0; i < n; i++) {
        stream = stream && gemv_use_stream(jobs[i].type, jobs[i].seq, cols);
        total_rows += (size_t)jobs[i].rows;
    }
    const int R = stream ? gs_pick_rows(total_rows, sm_count) : 0;
    int tile0 = 0;
    for (int i = 0; i < n; i++) {
        if (stream) jobs[i].rows_per_tile = R;
        jobs[i].tile0 = tile0;
        tile0 += (jobs[i].rows + jobs[i].rows_per_tile - 1) / jobs[i].rows_per_tile;
    }
}

inline int launch_quantize_q8k(cudaStream_t s, const float *x, size_t cols, size_t seq,
                               uint8_t *dev_out, uint8_t *ref_out) {
    const int nblk = (int)(cols / 256 * seq);
    if (nblk == 0) return RNB_B200_OK;
    RNB_CU(launch_k(quantize_q8k_kernel, dim3((nblk + 3) / 4), dim3(128), 0, s, x, (int)cols,
                    (int)seq, dev_out, ref_out));
    return RNB_B200_OK;
}

inline int flash_decode_default_chunks(size_t kv_len, size_t num_kv_heads, int sm_count) {
    if (kv_len == 0) return 1;
    static const bool per_sm_given = [] {
        const char *e = getenv("RNB_B200_FD_CTAS_PER_SM");
        return e && *e;
    }();
    static const int per_sm = [] {
        const char *e = getenv("RNB_B200_FD_CTAS_PER_SM");
        const int v = (e && *e) ? atoi(e) : 4;
        return v < 1 ? 1 : (v > 16 ? 16 : v);
    }();
    long want = (long)(per_sm * sm_count) / (long)(num_kv_heads ? num_kv_heads : 1);
    // The merge kernel's cost grows with the chunks per head, so short chunks do not pay: with four or
    // more KV heads on this GPU the count is held to max(SM / 2, kv_len / 128).  Measured: the
    // Llama-3-8B shape at 4096 and the 4-KV-head MoE shape at 8192 are fastest at 74 chunks per head
    // (MoE: 248 against 233 tok/s at 148); the 4-KV-head 70B shard at 32768 keeps its 148 (72.0
    // against 70.1 tok/s at 74).
    if (!per_sm_given && num_kv_heads >= 4) {
        const long cap = std::max<long>(sm_count / 2, (long)(kv_len / 128));
        if (want > cap) want = cap;
    }
    long max_c = (long)((kv_len + 31) / 32);
    if (want > max_c) want = max_c;
    if (want > FD_MAX_CHUNKS) want = FD_MAX_CHUNKS;
    if (want < 1) want = 1;
    return (int)want;
}
inline size_t flash_decode_scratch_bytes(size_t num_heads, int n_chunks) {
    return num_heads * (size_t)n_chunks * FD_PART_STRIDE * sizeof(float);
}
// Chunks per KV head when the attention kernel is launched as thread-block clusters that merge their
// own chunks (RNB_B200_ATTN_CLUSTER = 2..16; sixteen needs the non-portable cluster size opt-in), 0 if
// off or not schedulable.  Off by default: a cluster is at most 16 CTAs per KV head, and the Llama-3-8B
// shape at context 4096 wants about 74 (measured 2.52 ms per token with clusters of 16 against 2.24 ms
// with 74 chunks and a merge launch).
inline int flash_decode_cluster_size() {
    static const int v = [] {
        const char *e = getenv("RNB_B200_ATTN_CLUSTER");
        const int want = e && *e ? atoi(e) : 0;
        if (want < 2) return 0;
        if (cudaFuncSetAttribute(flash_decode_mma_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) cudaGetLastError();
        for (int c = want > 16 ? 16 : want; c >= 2; c /= 2) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(1, c);
            cfg.blockDim = dim3(FDM_THREADS);
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = c;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, flash_decode_mma_kernel, &cfg) == cudaSuccess && n > 0) return c;
            cudaGetLastError();
        }
        return 0;
    }();
    return v;
}
// Partial records of every (head, chunk).  f16 caches on 16-byte boundaries take the
// tensor-core kernel (its bulk copies need that alignment); anything else the CUDA-core one.
inline bool flash_decode_force_simt() {
    static const bool v = [] {
        const char *e = getenv("RNB_B200_FD_SIMT");
        return e && *e == '1';
    }();
    return v;
}
// `merge` (optional): let the tensor-core kernel's last CTA per KV head merge the chunks; *merged tells the
// caller whether that happened (it does not on the CUDA-core fallback) or a merge launch is still needed.
inline int launch_flash_decode_partials(cudaStream_t s, const float *q, const uint16_t *k, const uint16_t *v,
                                        const int *kv_len_dev, int kv_len_host, int num_heads, int num_kv_heads,
                                        float scale, float *partials, int n_chunks, int *dev_error, const FdMerge *merge = nullptr,
                                        bool *merged = nullptr) {
    const bool aligned = (((uintptr_t)k | (uintptr_t)v) & 15) == 0;
    if (merged) *merged = false;
    if (aligned && !flash_decode_force_simt()) {
        FdMerge m{nullptr, nullptr, nullptr, 0};
        const int group = num_kv_heads ? num_heads / num_kv_heads : 0;
        if (merge && merge->cluster > 0 && merge->cluster == n_chunks && 2 * n_chunks >= group && (!merge->xq_out || group % 2 == 0)) {
            // one cluster per KV head: its CTAs merge the chunks after a cluster barrier, no merge launch
            m = *merge;
            m.counters = nullptr;
            if (merged) *merged = true;
            RNB_CU(launch_k_cluster(flash_decode_mma_kernel, dim3(num_kv_heads, n_chunks), dim3(FDM_THREADS), 0, s, (unsigned)n_chunks, q, k, v, kv_len_dev,
                                    kv_len_host, num_heads, num_kv_heads, scale, partials, dev_error, m));
            return RNB_B200_OK;
        }
        if (merge && merge->counters && n_chunks <= FD_MAX_CHUNKS && (!merge->xq_out || group % 2 == 0)) {
            m = *merge;
            if (merged) *merged = true;
        }
        RNB_CU(launch_k(flash_decode_mma_kernel, dim3(num_kv_heads, n_chunks), dim3(FDM_THREADS), 0, s, q, k, v, kv_len_dev,
                        kv_len_host, num_heads, num_kv_heads, scale, partials, dev_error, m));
    } else
        RNB_CU(launch_k(flash_decode_partials_kernel, dim3(num_kv_heads, n_chunks), dim3(FD_THREADS), 0, s, q, k, v,
                        kv_len_dev, kv_len_host, num_heads, num_kv_heads, scale, partials));
    return RNB_B200_OK;
}
// kv_len = (*kv_len_dev if given) + kv_len_host
inline int launch_flash_decode(cudaStream_t s, const float *q, const uint16_t *k, const uint16_t *v,
                               const int *kv_len_dev, int kv_len_host, int num_heads,
                               int num_kv_heads, float scale, float *partials, int n_chunks,
                               float *out, int *dev_error = nullptr) {
    RNB_TRY(launch_flash_decode_partials(s, q, k, v, kv_len_dev, kv_len_host, num_heads, num_kv_heads, scale, partials,
                                         n_chunks, dev_error));
    RNB_CU(launch_k(flash_decode_reduce_kernel, dim3(num_heads), dim3(4 * HD), 0, s,
                    (const float *)partials, n_chunks, out, PeerOut{}));
    return RNB_B200_OK;
}

// Longest context the reference-order attention kernel serves (RNB_B200_EXACT_ATTN_MAX, default
// 512, at most 4096, 0 turns it off): up to there decode attention is bit-identical to rnb-cpu's; beyond it the
// chunked tensor-core kernel takes over, whose sums are reassociated.
inline int exact_attention_max() {
    static const int v = [] {
        const char *e = getenv("RNB_B200_EXACT_ATTN_MAX");
        long n = e && *e ? strtol(e, nullptr, 10) : 512;
        if (n < 0) n = 0;
        if (n > AX_MAX_LEN) n = AX_MAX_LEN;
        return (int)((n + 3) & ~3L);
    }();
    return v;
}
// raises the kernel's dynamic shared-memory limit once (not a stream operation: call it before a capture)
inline int attention_exact_setup() {
    static bool done = false;
    if (!done) {
        RNB_CU(cudaFuncSetAttribute(attention_decode_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ax_smem_bytes(AX_MAX_LEN)));
        done = true;
    }
    return RNB_B200_OK;
}
// kv_len = (*kv_len_dev if given) + kv_len_host must not exceed max_len (the kernel raises the error flag otherwise)
inline int launch_attention_decode_exact(cudaStream_t s, const float *q, const uint16_t *k, const uint16_t *v, const int *kv_len_dev,
                                         int kv_len_host, int max_len, int num_heads, int num_kv_heads, float scale, float *out,
                                         uint8_t *xq_out, int *dev_error) {
    if (max_len < 4 || max_len > AX_MAX_LEN || max_len % 4) return fail(RNB_B200_VALIDATION_FAILED, "exact attention: max_len %d must be a multiple of 4 in 4..%d", max_len, AX_MAX_LEN);
    if (xq_out && num_heads % 2) return fail(RNB_B200_VALIDATION_FAILED, "exact attention: Q8_K output needs an even head count");
    if (((uintptr_t)k | (uintptr_t)v) & 15u) return fail(RNB_B200_VALIDATION_FAILED, "exact attention: K and V must be 16-byte aligned");
    RNB_TRY(attention_exact_setup());
    RNB_CU(launch_k(attention_decode_exact_kernel, dim3((num_heads + 1) / 2), dim3(AX_THREADS), ax_smem_bytes(max_len), s, q, k, v,
                    kv_len_dev, kv_len_host, max_len, num_heads, num_kv_heads, scale, out, xq_out, dev_error));
    return RNB_B200_OK;
}
// Decode attention with the context length known on the host: reference-order kernel for short
// contexts, chunked kernel + merge otherwise.
inline int launch_attention_decode(cudaStream_t s, const float *q, const uint16_t *k, const uint16_t *v, int kv_len, int num_heads,
                                   int num_kv_heads, float scale, float *partials, int n_chunks, float *out, int *dev_error) {
    if (kv_len <= exact_attention_max() && ((((uintptr_t)k | (uintptr_t)v) & 15u) == 0))
        return launch_attention_decode_exact(s, q, k, v, nullptr, kv_len, (kv_len + 3) & ~3, num_heads, num_kv_heads, scale, out, nullptr, dev_error);
    return launch_flash_decode(s, q, k, v, nullptr, kv_len, num_heads, num_kv_heads, scale, partials, n_chunks, out, dev_error);
}

// Tensor-core prefill matmul: converts the f32 token rows to bf16 (scratch `xb`, seq*cols
// elements) and runs the tcgen05 kernel.  y is [seq][rows] f32.
int prefill_gemm_setup();   // raises the kernels' dynamic shared-memory limit once
// Descriptor of the bf16 token matrix [seq][cols] for the kernel's tiled copies: boxes of
// 64 columns x 256 tokens, 128-byte swizzle, zeros past the last token.  The encoder is a driver
// entry point, looked up once through the runtime.
inline int encode_token_map(PgTensorMap *out, const uint16_t *xb, size_t seq, size_t cols) {
    static_assert(sizeof(PgTensorMap) == sizeof(CUtensorMap) && alignof(PgTensorMap) >= alignof(CUtensorMap), "descriptor size");
    typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                    const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiled encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        RNB_CU(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !fn) return fail(RNB_B200_UNSUPPORTED, "the driver has no cuTensorMapEncodeTiled");
        encode = reinterpret_cast<EncodeTiled>(fn);
    }
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)seq};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)PG_K, (cuuint32_t)PG_BOX_ROWS};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(reinterpret_cast<CUtensorMap *>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t *>(xb), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(RNB_B200_CUDA_ERROR, "cuTensorMapEncodeTiled failed with driver code %d", (int)r);
    return RNB_B200_OK;
}
inline int launch_prefill_gemm_multi(cudaStream_t s, int n, const int *types, const uint8_t *const *w, const size_t *rows, float *const *y,
                                     size_t cols, const float *x, size_t seq, uint16_t *xb, int *dev_error) {
    if (n < 1 || n > PG_MAX_JOBS) return fail(RNB_B200_VALIDATION_FAILED, "prefill matmul takes 1..%d matrices per launch", PG_MAX_JOBS);
    if (cols == 0 || cols % 256 != 0) return fail(RNB_B200_VALIDATION_FAILED, "cols(%zu) must be a non-zero multiple of 256", cols);
    if (seq == 0) return fail(RNB_B200_VALIDATION_FAILED, "prefill matmul needs tokens");
    if (((uintptr_t)x & 15u) || ((uintptr_t)xb & 15u)) return fail(RNB_B200_VALIDATION_FAILED, "prefill matmul operands are not aligned");
    // x == nullptr: `xb` already holds the bf16 token matrix (written by the producer of the activation)
    PgJobs jobs;
    memset(&jobs, 0, sizeof(jobs));
    jobs.n = n;
    int tiles = 0;
    for (int i = 0; i < n; i++) {
        if (types[i] != TYPE_Q4_K && types[i] != TYPE_Q6_K) return fail(RNB_B200_UNSUPPORTED, "tensor-core prefill matmul supports Q4_K and Q6_K weights");
        if (rows[i] == 0) return fail(RNB_B200_VALIDATION_FAILED, "prefill matmul needs rows");
        if (((uintptr_t)w[i] & 1u) || ((uintptr_t)y[i] & 15u) || (types[i] == TYPE_Q4_K && ((uintptr_t)w[i] & 15u)))
            return fail(RNB_B200_VALIDATION_FAILED, "prefill matmul operands are not aligned");
        jobs.j[i].w = w[i];
        jobs.j[i].y = y[i];
        jobs.j[i].rows = (int)rows[i];
        jobs.j[i].type = types[i];
        jobs.j[i].tile0 = tiles;
        tiles += (int)((rows[i] + PG_ROWS - 1) / PG_ROWS);
    }
    RNB_TRY(prefill_gemm_setup());
    const size_t ne = seq * cols;
    if (x) RNB_CU(launch_k(f32_to_bf16_kernel, dim3((unsigned)((ne / 8 + 255) / 256)), dim3(256), 0, s, x, xb, ne));
    PgTensorMap tmap;
    RNB_TRY(encode_token_map(&tmap, xb, seq, cols));
    const dim3 grid((unsigned)tiles, (unsigned)((seq + PG_TOK - 1) / PG_TOK));
    RNB_CU(launch_k(prefill_gemm_kernel, grid, dim3(PG_THREADS), PG_SMEM, s, jobs, tmap, (int)seq, (int)cols, dev_error));
    return RNB_B200_OK;
}
// gate + up of a token batch with silu(gate) * up in the epilogue: act [seq][rows] bf16, ready to be the token matrix of
// the down matmul.  `act` must not alias `xb` (other CTAs are still reading tokens when the first tiles finish).
inline int launch_prefill_gemm_silu(cudaStream_t s, int type, const uint8_t *gate, const uint8_t *up, size_t rows, size_t cols, const float *x, size_t seq,
                                    uint16_t *xb, uint16_t *act, int *dev_error) {
    if (type != TYPE_Q4_K && type != TYPE_Q6_K) return fail(RNB_B200_UNSUPPORTED, "tensor-core prefill matmul supports Q4_K and Q6_K weights");
    if (cols == 0 || cols % 256 != 0) return fail(RNB_B200_VALIDATION_FAILED, "cols(%zu) must be a non-zero multiple of 256", cols);
    if (seq == 0 || rows == 0) return fail(RNB_B200_VALIDATION_FAILED, "prefill matmul needs tokens and rows");
    if (!gate || !up || !xb || !act || act == xb) return fail(RNB_B200_VALIDATION_FAILED, "prefill gate+up: null or aliased operands");
    if (((uintptr_t)x & 15u) || ((uintptr_t)xb & 15u) || ((uintptr_t)act & 1u) || (((uintptr_t)gate | (uintptr_t)up) & (type == TYPE_Q4_K ? 15u : 1u)))
        return fail(RNB_B200_VALIDATION_FAILED, "prefill matmul operands are not aligned");
    PgJobs jobs;
    memset(&jobs, 0, sizeof(jobs));
    jobs.n = 1;
    jobs.j[0].w = gate;
    jobs.j[0].w2 = up;
    jobs.j[0].yb = act;
    jobs.j[0].rows = (int)rows;
    jobs.j[0].type = type;
    const int tiles = (int)((rows + PG_ROWS / 2 - 1) / (PG_ROWS / 2));
    RNB_TRY(prefill_gemm_setup());
    const size_t ne = seq * cols;
    if (x) RNB_CU(launch_k(f32_to_bf16_kernel, dim3((unsigned)((ne / 8 + 255) / 256)), dim3(256), 0, s, x, xb, ne));
    PgTensorMap tmap;
    RNB_TRY(encode_token_map(&tmap, xb, seq, cols));
    const dim3 grid((unsigned)tiles, (unsigned)((seq + PG_TOK - 1) / PG_TOK));
    RNB_CU(launch_k(prefill_gemm_kernel, grid, dim3(PG_THREADS), PG_SMEM, s, jobs, tmap, (int)seq, (int)cols, dev_error));
    return RNB_B200_OK;
}
inline int launch_prefill_gemm(cudaStream_t s, int type, const uint8_t *w, size_t rows, size_t cols, const float *x, size_t seq,
                               uint16_t *xb, float *y, int *dev_error) {
    return launch_prefill_gemm_multi(s, 1, &type, &w, &rows, &y, cols, x, seq, xb, dev_error);
}

}  // namespace rnb
