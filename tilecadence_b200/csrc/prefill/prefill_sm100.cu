// Causal GQA prefill (four query heads per KV head, D = 128, BF16) for sm_100a: O and LSE.
//
// Path replaced: tilecadence/cuda/prefill/prefill.cu:21-43,122-152 (CTA mapping, host checks,
// launch), long_prefill_rowblock.cuh:117-605 (the row-block kernel: QK^T, online softmax with a
// gated rescale :68-115, PV, O staged in shared memory for 16-byte stores :513-524, both heads' LSE staged
// in the released terminal K span :539-587) and common.cuh:36-78 (tensor checks).
//
// A unit of work is a 128-row query tile of the two query heads that share a KV head pair slot, so one
// K/V tile in shared memory feeds both heads. Two schedules of the same pipeline: for sequences of up to
// 4096 tokens one persistent CTA per SM works through a list of units dealt from the longest-first order,
// the loads and the first MMAs of a unit overlapping the epilogue of the unit before it (prefill_kernel);
// for longer ones the grid holds one CTA per unit, longest first (prefill_rowblock_kernel). What follows
// describes the persistent form. The two dense contractions run on the 5th-generation
// tensor cores: S = Q_h K^T as a shared x shared tcgen05.mma into one 128-column score buffer in TMEM
// that the two heads use in strict alternation, O_h += P_h V as a TMEM x shared tcgen05.mma with P_h
// (BF16) in columns of its own. TMEM: S | P0 P1 | O0 | O1 = 128 + 2*64 + 2*128 = all 512 columns. Roles:
//   warps 0-3  softmax for head 0 (one query row per thread, TMEM lane = row)
//   warps 4-7  softmax for head 1
//   warp  8    TMA producer: Q of each unit, a 2-stage K ring and a 2-stage V ring (128-byte swizzle)
//   warp  9    issues every score MMA (one elected thread; the warp also owns TMEM)
//   warps 10,11 issue PV for head 0 / head 1 (one elected thread each)
// The third warpgroup gives most of its registers to the softmax warpgroups (setmaxnreg). Score
// MMAs and PV MMAs have separate issuers because issue blocks at the tensor pipe's rate: a thread that
// is busy issuing one kind must not be the one that has to notice the other kind becoming ready. The
// softmax is bound by the exponential unit (16 results per clock per SM against 8192 MMA flops), so
// the two warpgroups take turns at it (named barriers). A head may rewrite the first half of its P as
// soon as the first half of the previous PV has retired. Key tiles go from the diagonal down to 0; the
// ring index is chosen so that a unit's final tile always uses stage 0: that stage is the "terminal K" donor
// whose bytes receive the two 512-byte LSE arrays as soon as the unit's last softmax is done. The BF16 output
// tile of a head leaves through a 32 KiB staging buffer that the two heads use in turn.
#include "config.cuh"
#include "tc_host.cuh"
#include "tc_ptx.cuh"

#include <cmath>

namespace {

constexpr int kBlockM = PREFILL_BLOCK_M;
constexpr int kBlockN = PREFILL_BLOCK_N;
constexpr int kDim = 128;
constexpr int kGroup = 4;
constexpr int kStages = PREFILL_KV_STAGES;
constexpr int kTileBytes = 128 * kDim * 2;    // one 128-row operand tile
constexpr int kHalfBytes = kTileBytes / 2;    // 64 of the 128 head-dim elements, all rows
constexpr int kQOffset = 0;
constexpr int kKOffset = 2 * kTileBytes;
constexpr int kVOffset = kKOffset + kStages * kTileBytes;
constexpr int kBarrierBytes = 256;
constexpr int kStagingBytes = 1024;           // dedicated LSE staging when the handoff is disabled
constexpr int kSoftmaxThreads = 128;
constexpr int kThreads = 3 * kSoftmaxThreads;   // two softmax warpgroups + one data/MMA warpgroup
constexpr int kSoftmaxRegisters = 216, kDataRegisters = 72;  // 256*216 + 128*72 = 64512 <= 65536
constexpr int kProducerWarp = 8, kMmaWarp = 9;
// Tensor-memory map, solved by the planner (placement.TMEM_MAPS["prefill"]) and emitted into config.cuh.
constexpr uint32_t kTmemColumns = PREFILL_TMEM_ALLOCATION_COLUMNS;
constexpr uint32_t kSColumns = 128, kPColumns = 64, kOColumns = 128;  // FP32 scores, BF16 pairs, FP32 output
__host__ __device__ constexpr uint32_t s_column(int h) { return h == 0 ? PREFILL_TMEM_S_HEAD0_COLUMN : PREFILL_TMEM_S_HEAD1_COLUMN; }
__host__ __device__ constexpr uint32_t p_column(int h) { return h == 0 ? PREFILL_TMEM_P_HEAD0_COLUMN : PREFILL_TMEM_P_HEAD1_COLUMN; }
__host__ __device__ constexpr uint32_t o_column(int h) { return h == 0 ? PREFILL_TMEM_O_HEAD0_COLUMN : PREFILL_TMEM_O_HEAD1_COLUMN; }
constexpr bool columns_disjoint(uint32_t a, uint32_t a_columns, uint32_t b, uint32_t b_columns) {
    return a + a_columns <= b || b + b_columns <= a;
}
constexpr float kRescaleThreshold = 8.f;      // log2 units: P stays below 2^8

static_assert(kBlockM == 128 && kBlockN == 128 && PREFILL_GROUP_HEADS == 2 && kStages == 2, "fixed tile schedule");
static_assert(kTmemColumns >= 32 && kTmemColumns <= 512 && (kTmemColumns & (kTmemColumns - 1)) == 0,
              "a tensor-memory allocation is a power of two between 32 and 512 columns");
static_assert(s_column(0) % 32 == 0 && s_column(1) % 32 == 0 && o_column(0) % 32 == 0 && o_column(1) % 32 == 0 &&
                  p_column(0) % 16 == 0 && p_column(1) % 16 == 0, "tile column alignment");
static_assert(s_column(0) + kSColumns <= kTmemColumns && s_column(1) + kSColumns <= kTmemColumns &&
                  p_column(0) + kPColumns <= kTmemColumns && p_column(1) + kPColumns <= kTmemColumns &&
                  o_column(0) + kOColumns <= kTmemColumns && o_column(1) + kOColumns <= kTmemColumns,
              "tiles must lie inside the allocation");
// The score buffers of the two heads are never alive together (the kernel hands them over 0,1,0,1,...), so
// they may coincide; if they do not coincide they must not partly overlap. Everything else is alive together.
static_assert(s_column(0) == s_column(1) || columns_disjoint(s_column(0), kSColumns, s_column(1), kSColumns),
              "score buffers are either one shared buffer or disjoint");
static_assert(columns_disjoint(p_column(0), kPColumns, p_column(1), kPColumns) &&
                  columns_disjoint(o_column(0), kOColumns, o_column(1), kOColumns),
              "per-head probability and output tiles must not overlap");
static_assert(columns_disjoint(s_column(0), kSColumns, p_column(0), kPColumns) && columns_disjoint(s_column(0), kSColumns, p_column(1), kPColumns) &&
                  columns_disjoint(s_column(1), kSColumns, p_column(0), kPColumns) && columns_disjoint(s_column(1), kSColumns, p_column(1), kPColumns) &&
                  columns_disjoint(s_column(0), kSColumns, o_column(0), kOColumns) && columns_disjoint(s_column(0), kSColumns, o_column(1), kOColumns) &&
                  columns_disjoint(s_column(1), kSColumns, o_column(0), kOColumns) && columns_disjoint(s_column(1), kSColumns, o_column(1), kOColumns) &&
                  columns_disjoint(p_column(0), kPColumns, o_column(0), kOColumns) && columns_disjoint(p_column(0), kPColumns, o_column(1), kOColumns) &&
                  columns_disjoint(p_column(1), kPColumns, o_column(0), kOColumns) && columns_disjoint(p_column(1), kPColumns, o_column(1), kOColumns),
              "score, probability and output tiles are alive together and must not overlap");
static_assert(PREFILL_TERMINAL_K_OFFSET_BYTES == kKOffset && PREFILL_TERMINAL_K_BYTES == kTileBytes,
              "the planner's donor must be K stage 0");
static_assert(PREFILL_LSE_HEAD0_OFFSET_BYTES % 128 == 0 && PREFILL_LSE_HEAD1_OFFSET_BYTES % 128 == 0, "alignment");
static_assert(PREFILL_LSE_HEAD0_OFFSET_BYTES >= kKOffset && PREFILL_LSE_HEAD0_OFFSET_BYTES + 512 <= kKOffset + kTileBytes &&
                  PREFILL_LSE_HEAD1_OFFSET_BYTES >= kKOffset &&
                  PREFILL_LSE_HEAD1_OFFSET_BYTES + 512 <= kKOffset + kTileBytes,
              "LSE regions must lie inside the terminal K stage");
static_assert(PREFILL_LSE_HEAD0_OFFSET_BYTES + 512 <= PREFILL_LSE_HEAD1_OFFSET_BYTES ||
                  PREFILL_LSE_HEAD1_OFFSET_BYTES + 512 <= PREFILL_LSE_HEAD0_OFFSET_BYTES,
              "LSE regions must not overlap");

constexpr int kOutStageOffset = kVOffset + kStages * kTileBytes;  // one 128 x 128 BF16 tile, used by the heads in turn
constexpr int kBarrierOffset = kOutStageOffset + kTileBytes;
constexpr int shared_bytes(bool handoff) { return 1024 + kBarrierOffset + kBarrierBytes + (handoff ? 0 : kStagingBytes); }
static_assert(shared_bytes(false) <= 227 * 1024, "the schedule must fit the 227 KiB a CTA can have");

struct Barriers {
    uint64_t q_full, q_empty;
    uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
    uint64_t s_full[2], s_free[2], p_half[2][2], p_lo_free[2], o_done[2];
    uint64_t o_free[2];          // the epilogue has read head h's accumulator out of tensor memory
    uint64_t lse_drained;        // both heads' LSE arrays have left the terminal K stage
    uint64_t stage_drained[2];   // head h's output tile has left the staging buffer
    uint32_t tmem_base;
    int32_t abort;
    int32_t role[2];  // key-split only: which of the two CTAs of a query tile claimed each head first
};
static_assert(sizeof(Barriers) <= kBarrierBytes, "barrier block");

struct PrefillParams {
    float* lse;
    int32_t* status;
    int batch, tokens, q_heads, kv_heads, m_blocks;
    int total_units;  // work units of the launch: (query tile, batch, KV head, head pair[, key part]), longest first
    float scale, scale_log2;
    // Key-split launches only: per (query tile, head) a claim counter and a ready word (zeroed before the
    // launch), 128 x 128 normalised fp32 O values stored as [32 column groups][128 rows] float4, 128 LSEs.
    int32_t* tickets;
    float4* part_o;
    float* part_lse;
};

__device__ __forceinline__ void wg_barrier(int head) {
    asm volatile("bar.sync %0, %1;" ::"r"(head + 1), "n"(kSoftmaxThreads) : "memory");
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Uses of the two ring stages so far, kept in two registers (an indexed array would live in local memory).
struct StageCounts {
    uint32_t stage0 = 0, stage1 = 0;
    __device__ __forceinline__ uint32_t of(int stage) const { return stage == 0 ? stage0 : stage1; }
    __device__ __forceinline__ void bump(int stage) {
        if (stage == 0) ++stage0; else ++stage1;
    }
};
static_assert(kStages == 2, "StageCounts holds two stages");

// One unit of work: a 128-row query tile of the two heads of a pair slot and the key tiles it attends to
// (all of them, or with kSplit one of two parts: part 0 the tiles nearest the diagonal, rounded up).
struct Unit {
    int m_block, part, pair, kvh, b, head0, m0, all_tiles, n_tiles, key_block0;
};
template <bool kSplit>
__device__ __forceinline__ Unit unit_at(const PrefillParams& p, int index) {
    // Longest query tiles first; neighbouring units share a KV head so K/V tiles hit in L2.
    Unit u;
    const int per_block = p.batch * p.kv_heads * 2 * (kSplit ? 2 : 1);
    u.m_block = p.m_blocks - 1 - index / per_block;
    int rest = index % per_block;
    u.part = kSplit ? (rest & 1) : 0;
    if (kSplit) rest >>= 1;
    u.pair = rest & 1;
    u.kvh = (rest >> 1) % p.kv_heads;
    u.b = rest / (2 * p.kv_heads);
    u.head0 = u.kvh * kGroup + u.pair * 2;
    u.m0 = u.m_block * kBlockM;
    // Key tiles m_block, m_block-1, ..., 0; this unit's share is n_tiles of them starting at key_block0.
    u.all_tiles = u.m_block + 1;
    const int near_tiles = kSplit ? (u.all_tiles + 1) / 2 : u.all_tiles;
    u.n_tiles = u.part == 0 ? near_tiles : u.all_tiles - near_tiles;
    u.key_block0 = u.part == 0 ? u.m_block : u.m_block - near_tiles;
    return u;
}
// Units are dealt to the CTAs of the (persistent) grid in rounds that change direction, so that every CTA gets
// a similar amount of work from the sorted list. Returns -1 when the round has no unit for this CTA.
__device__ __forceinline__ int unit_of_round(int round, int total_units) {
    const int grid = int(gridDim.x), cta = int(blockIdx.x);
    const int index = round * grid + ((round & 1) ? grid - 1 - cta : cta);
    return index < total_units ? index : -1;
}

// Build switch TC_TRACE (off in every shipped library): one thread of each role appends (tag, %globaltimer) records
// to a per-CTA, per-role log that tc_debug_prefill_trace copies out; see tilecadence_b200/trace_prefill.py.
// Roles: 0 TMA producer, 1 score-MMA issuer, 2/3 PV issuers, 4/5 softmax warpgroups (row 0).
// Tags: 1 Q tiles issued, 2 first K/V tile of a unit issued, 3 last tile of a unit issued; 10 first / 11 last score
// MMA of a unit issued; 20 first / 21 last PV of a unit issued; 30 first score tile of a unit arrived, 31 key loop
// done, 32 LSE array left, 33 last PV done, 34 output tile left.
#ifdef TC_TRACE
constexpr int kTraceRoles = 6, kTraceEvents = 256;
__device__ unsigned long long g_prefill_trace[148][kTraceRoles][kTraceEvents];
#define TC_TRACE_DECLARE(role) unsigned long long* trace_log = blockIdx.x < 148 ? g_prefill_trace[blockIdx.x][role] : nullptr; int trace_count = 0
#define TC_TRACE_EVENT(tag) do { if (trace_log && trace_count < kTraceEvents) trace_log[trace_count++] = (tc::global_timer_ns() << 8) | (unsigned long long)(tag); } while (0)
#else
#define TC_TRACE_DECLARE(role) do { } while (0)
#define TC_TRACE_EVENT(tag) do { } while (0)
#endif

// Persistent kernel: one CTA per SM works through its units. Barrier phases run on across units (every waiter
// sees every phase of the barriers it waits on, in order, and keeps its own count), so the TMA producer and the
// MMA issuers move on to the next unit while the softmax warpgroups are still in the epilogue of the current
// one: Q of the next unit is loaded as soon as the last score MMA has read the current Q, K/V tiles as soon as
// ring stages are free, and the first score MMA of the next unit is issued as soon as the score buffer is.
// kSplit: two units per query tile (see Unit); whichever CTA finishes a head second merges the other's
// normalised O and LSE into its own (LSE-weighted) and stores. For launches whose query tiles are too few to
// fill the GPU, where the longest tile alone would set the run time.
template <bool kHandoff, bool kSplit = false>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
               const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap omap,
               const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(smem + kBarrierOffset);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rounds = (p.total_units + int(gridDim.x) - 1) / int(gridDim.x);

    int preissued_tiles = -1;  // producer thread: tiles of the first unit already sent for (-1: nor its Q)
    if (threadIdx.x == kProducerWarp * 32) {
        tc::mbar_init(&bars->q_full, 1);
        tc::mbar_init(&bars->q_empty, 1);
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(&bars->k_full[s], 1);
            tc::mbar_init(&bars->k_empty[s], 2);  // one arrival per head's score MMA
            tc::mbar_init(&bars->v_full[s], 1);
            tc::mbar_init(&bars->v_empty[s], 2);  // one arrival per head's PV issuer
        }
        tc::mbar_init(&bars->lse_drained, 2);
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&qmap);
        tc::tma_prefetch_desc(&kmap);
        tc::tma_prefetch_desc(&vmap);
        // The operand barriers are this thread's own, and the stages are fresh: Q and the first ring stages of the
        // CTA's first unit are sent for at once, so that they fly while the other warps set up their barriers and
        // tensor memory. Everything else waits for the CTA barrier below.
        const Unit first = unit_at<kSplit>(p, unit_of_round(0, p.total_units));
        if (first.n_tiles > 0) {
            const uint64_t keep = tc::policy_evict_last(), stream_once = tc::policy_evict_first();
            tc::mbar_arrive_expect_tx(&bars->q_full, 2 * kTileBytes);
            for (int h = 0; h < 2; ++h) {
                uint8_t* dst = smem + kQOffset + h * kTileBytes;
                tc::tma_load_4d(dst, &qmap, &bars->q_full, 0, first.head0 + h, first.m0, first.b, stream_once);
                tc::tma_load_4d(dst + kHalfBytes, &qmap, &bars->q_full, 64, first.head0 + h, first.m0, first.b, stream_once);
            }
            preissued_tiles = first.n_tiles < kStages ? first.n_tiles : kStages;
            for (int it = 0; it < preissued_tiles; ++it) {
                const int stage = (first.n_tiles - 1 - it) % kStages;
                const int n0 = (first.key_block0 - it) * kBlockN;
                uint8_t* kdst = smem + kKOffset + stage * kTileBytes;
                tc::mbar_arrive_expect_tx(&bars->k_full[stage], kTileBytes);
                tc::tma_load_4d(kdst, &kmap, &bars->k_full[stage], 0, first.kvh, n0, first.b, keep);
                tc::tma_load_4d(kdst + kHalfBytes, &kmap, &bars->k_full[stage], 64, first.kvh, n0, first.b, keep);
                uint8_t* vdst = smem + kVOffset + stage * kTileBytes;
                tc::mbar_arrive_expect_tx(&bars->v_full[stage], kTileBytes);
                tc::tma_load_4d(vdst, &vmap, &bars->v_full[stage], 0, first.kvh, n0, first.b, keep);
                tc::tma_load_4d(vdst + kHalfBytes, &vmap, &bars->v_full[stage], 64, first.kvh, n0, first.b, keep);
            }
        }
    }
    if (threadIdx.x == 0) {
        for (int h = 0; h < 2; ++h) {
            tc::mbar_init(&bars->s_full[h], 1);
            tc::mbar_init(&bars->s_free[h], kSoftmaxThreads);
            tc::mbar_init(&bars->p_half[h][0], kSoftmaxThreads);
            tc::mbar_init(&bars->p_half[h][1], kSoftmaxThreads);
            tc::mbar_init(&bars->o_done[h], 1);
            tc::mbar_init(&bars->p_lo_free[h], 1);
            tc::mbar_init(&bars->o_free[h], kSoftmaxThreads);
            tc::mbar_init(&bars->stage_drained[h], 1);
        }
        bars->abort = 0;
        tc::mbar_fence_init();
    }
    if (warp == kMmaWarp) {
        tc::tmem_alloc(&bars->tmem_base, kTmemColumns);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem = bars->tmem_base;

    // The third warpgroup only moves data and issues MMAs: it hands most of its registers to the
    // two softmax warpgroups, which keep a whole 128-column score row per thread. Each role's code
    // sits under its own setmaxnreg so that the register allocator sees the right budget.
    if (warp >= 2 * (kSoftmaxThreads / 32)) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kDataRegisters));
    if (warp == kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint64_t keep = tc::policy_evict_last(), stream_once = tc::policy_evict_first();
            StageCounts k_uses, v_uses;  // loads issued into each ring stage so far
            uint32_t units_done = 0;
            bool ok = true;
            TC_TRACE_DECLARE(0);
            for (int round = 0; ok && round < rounds; ++round) {
                const int index = unit_of_round(round, p.total_units);
                if (index < 0) continue;
                const Unit u = unit_at<kSplit>(p, index);
                if (u.n_tiles == 0) continue;  // a one-tile row block has nothing to split
                int first_tile = 0;
                if (units_done == 0 && preissued_tiles >= 0) {
                    // The CTA's first unit: Q and the first ring stages were sent for before the CTA barrier.
                    first_tile = preissued_tiles;
                    for (int it = 0; it < preissued_tiles; ++it) {
                        k_uses.bump((u.n_tiles - 1 - it) % kStages);
                        v_uses.bump((u.n_tiles - 1 - it) % kStages);
                    }
                } else {
                    // Q: the score MMAs of the previous unit must have read the previous Q.
                    if (units_done > 0 && !(ok = tc::mbar_wait(&bars->q_empty, (units_done - 1) & 1))) break;
                    tc::mbar_arrive_expect_tx(&bars->q_full, 2 * kTileBytes);
                    for (int h = 0; h < 2; ++h) {
                        uint8_t* dst = smem + kQOffset + h * kTileBytes;
                        tc::tma_load_4d(dst, &qmap, &bars->q_full, 0, u.head0 + h, u.m0, u.b, stream_once);
                        tc::tma_load_4d(dst + kHalfBytes, &qmap, &bars->q_full, 64, u.head0 + h, u.m0, u.b, stream_once);
                    }
                }
                TC_TRACE_EVENT(1);
                bool terminal_checked = units_done == 0;
                for (int it = first_tile; it < u.n_tiles; ++it) {
                    const int stage = (u.n_tiles - 1 - it) % kStages;  // the unit's last tile always lands in stage 0
                    const int n0 = (u.key_block0 - it) * kBlockN;
                    if (k_uses.of(stage) > 0 && !(ok = tc::mbar_wait(&bars->k_empty[stage], (k_uses.of(stage) - 1) & 1))) break;
                    if (stage == 0 && !terminal_checked) {
                        // Stage 0 was the previous unit's terminal K stage: its LSE arrays must have left it.
                        if (!(ok = tc::mbar_wait(&bars->lse_drained, (units_done - 1) & 1))) break;
                        terminal_checked = true;
                    }
                    uint8_t* kdst = smem + kKOffset + stage * kTileBytes;
                    tc::mbar_arrive_expect_tx(&bars->k_full[stage], kTileBytes);
                    tc::tma_load_4d(kdst, &kmap, &bars->k_full[stage], 0, u.kvh, n0, u.b, keep);
                    tc::tma_load_4d(kdst + kHalfBytes, &kmap, &bars->k_full[stage], 64, u.kvh, n0, u.b, keep);
                    k_uses.bump(stage);
                    if (v_uses.of(stage) > 0 && !(ok = tc::mbar_wait(&bars->v_empty[stage], (v_uses.of(stage) - 1) & 1))) break;
                    uint8_t* vdst = smem + kVOffset + stage * kTileBytes;
                    tc::mbar_arrive_expect_tx(&bars->v_full[stage], kTileBytes);
                    tc::tma_load_4d(vdst, &vmap, &bars->v_full[stage], 0, u.kvh, n0, u.b, keep);
                    tc::tma_load_4d(vdst + kHalfBytes, &vmap, &bars->v_full[stage], 64, u.kvh, n0, u.b, keep);
                    v_uses.bump(stage);
                    if (it == 0) TC_TRACE_EVENT(2);
                    if (it + 1 == u.n_tiles) TC_TRACE_EVENT(3);
                }
                ++units_done;
            }
            if (!ok) {
                atomicCAS(p.status, 0, 11);
                bars->abort = 1;
            }
        }
    } else {
        // ------------------------------------------------------------------ MMA issuers
        // Warp 9 issues every score MMA (the shared score buffer is used 0,1,0,1,... so their order is
        // fixed anyway); warps 10 and 11 issue PV for head 0 and head 1. Each role is one elected thread.
        // Issue blocks at the tensor pipe's rate and every barrier check costs such a lone thread
        // 100-170 cycles, so a thread that is busy issuing one kind of MMA must not be the one that has
        // to notice that the other kind has become ready.
        if (lane == 0) {
            constexpr uint32_t idesc_qk = tc::umma_idesc(128, 128, 1, 0, 0);
            constexpr uint32_t idesc_pv = tc::umma_idesc(128, 128, 1, 0, 1);
            StageCounts uses;  // tiles taken from each ring stage so far (K for warp 9, V for 10 and 11)
            uint32_t tiles_done = 0, units_done = 0;
            bool ok = true;
            TC_TRACE_DECLARE(warp - kMmaWarp + 1);
            if (warp == kMmaWarp) {
                // S = Q_h K^T into the score buffer: both operands K-major, 8 steps of 16 along D
                // (4 per 64-element half). A score MMA may overwrite the buffer once the other head's
                // softmax warpgroup has pulled its tile into registers; because P has its own columns it
                // does not wait for any PV.
                const uint32_t q_addr = tc::smem_u32(smem + kQOffset);
                const uint32_t k_addr = tc::smem_u32(smem + kKOffset);
                for (int round = 0; ok && round < rounds; ++round) {
                    const int index = unit_of_round(round, p.total_units);
                    if (index < 0) continue;
                    const Unit u = unit_at<kSplit>(p, index);
                    if (u.n_tiles == 0) continue;
                    if (!(ok = tc::mbar_wait(&bars->q_full, units_done & 1))) break;
                    for (int it = 0; ok && it < u.n_tiles; ++it) {
                        const int stage = (u.n_tiles - 1 - it) % kStages;
                        if (!(ok = tc::mbar_wait(&bars->k_full[stage], uses.of(stage) & 1))) break;
                        uses.bump(stage);
                        const uint32_t kb = k_addr + stage * kTileBytes;
                        for (int h = 0; h < 2 && ok; ++h) {
                            if (h == 0) {
                                if (tiles_done > 0) ok = tc::mbar_wait(&bars->s_free[1], (tiles_done - 1) & 1);
                            } else {
                                ok = tc::mbar_wait(&bars->s_free[0], tiles_done & 1);
                            }
                            if (!ok) break;
                            tc::tc_fence_after_sync();
#pragma unroll
                            for (int ks = 0; ks < 8; ++ks) {
                                const uint32_t off = uint32_t(ks >> 2) * kHalfBytes + uint32_t(ks & 3) * 32;
                                tc::umma_ss(tmem + s_column(h), tc::umma_desc_sw128(q_addr + h * kTileBytes + off, 16, 1024),
                                            tc::umma_desc_sw128(kb + off, 16, 1024), idesc_qk, ks > 0);
                            }
                            tc::umma_commit(&bars->s_full[h]);
                            tc::umma_commit(&bars->k_empty[stage]);  // two arrivals per stage: one per head
                            if (it == 0 && h == 0) TC_TRACE_EVENT(10);
                            if (it + 1 == u.n_tiles && h == 1) TC_TRACE_EVENT(11);
                        }
                        ++tiles_done;
                    }
                    if (ok) tc::umma_commit(&bars->q_empty);  // every score MMA of this unit has read Q
                    ++units_done;
                }
            } else {
                // O_h += P_h V, one 64-key half at a time: P from TMEM (8 columns per 16 keys), V MN-major
                // (row = key, 128 bytes per 64 d; the d halves 16 KiB apart, 8-key groups 1 KiB).
                const int h = warp - (kMmaWarp + 1);
                const uint32_t v_addr = tc::smem_u32(smem + kVOffset);
                const uint32_t p_col = tmem + p_column(h);
                const uint32_t o_col = tmem + o_column(h);
                for (int round = 0; ok && round < rounds; ++round) {
                    const int index = unit_of_round(round, p.total_units);
                    if (index < 0) continue;
                    const Unit u = unit_at<kSplit>(p, index);
                    if (u.n_tiles == 0) continue;
                    for (int it = 0; ok && it < u.n_tiles; ++it) {
                        const int stage = (u.n_tiles - 1 - it) % kStages;
                        const uint32_t vb = v_addr + stage * kTileBytes;
                        auto issue_pv_half = [&](int half) {
#pragma unroll
                            for (int k4 = 0; k4 < 4; ++k4) {
                                const int ks = half * 4 + k4;
                                tc::umma_ts(o_col, p_col + uint32_t(ks) * 8, tc::umma_desc_sw128(vb + ks * 2048, kHalfBytes, 1024),
                                            idesc_pv, !(it == 0 && ks == 0));
                            }
                        };
                        if (!(ok = tc::mbar_wait(&bars->v_full[stage], uses.of(stage) & 1))) break;
                        uses.bump(stage);
                        // The first PV of a unit overwrites the accumulator: the previous unit's epilogue must
                        // have read it out of tensor memory.
                        if (it == 0 && units_done > 0 && !(ok = tc::mbar_wait(&bars->o_free[h], (units_done - 1) & 1))) break;
                        if (!(ok = tc::mbar_wait(&bars->p_half[h][0], tiles_done & 1))) break;
                        tc::tc_fence_after_sync();
                        issue_pv_half(0);
                        tc::umma_commit(&bars->p_lo_free[h]);  // P columns of the first 64 keys may be rewritten
                        if (!(ok = tc::mbar_wait(&bars->p_half[h][1], tiles_done & 1))) break;
                        tc::tc_fence_after_sync();
                        issue_pv_half(1);
                        tc::umma_commit(&bars->o_done[h]);
                        tc::umma_commit(&bars->v_empty[stage]);
                        if (it == 0) TC_TRACE_EVENT(20);
                        if (it + 1 == u.n_tiles) TC_TRACE_EVENT(21);
                        ++tiles_done;
                    }
                    ++units_done;
                }
            }
            if (!ok) {
                atomicCAS(p.status, 0, 13);
                bars->abort = 1;
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegisters));
        // ------------------------------------------------------------------ softmax warpgroups
        const int h = warp >> 2;                        // head slot
        const int row = threadIdx.x & (kSoftmaxThreads - 1);
        const uint32_t lane_field = uint32_t((warp & 3) * 32) << 16;
        const uint32_t s_tmem = tmem + lane_field + s_column(h);
        const uint32_t p_tmem = tmem + lane_field + p_column(h);
        const uint32_t o_tmem = tmem + lane_field + o_column(h);
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
        // Tiles of all of this CTA's units: the two heads take turns at the exponential unit from the first tile
        // of the first unit to the last tile of the last one.
        uint32_t cta_tiles = 0;
        for (int round = 0; round < rounds; ++round) {
            const int index = unit_of_round(round, p.total_units);
            if (index >= 0) cta_tiles += uint32_t(unit_at<kSplit>(p, index).n_tiles);
        }
        uint32_t tiles_done = 0, units_done = 0, terminal_uses = 0;  // terminal_uses: tiles that went through K stage 0
        bool ok = true;
#ifdef TC_TRACE
        unsigned long long* trace_log = (row == 0 && blockIdx.x < 148) ? g_prefill_trace[blockIdx.x][4 + h] : nullptr;
        int trace_count = 0;
#endif

        for (int round = 0; round < rounds; ++round) {
        const int index = unit_of_round(round, p.total_units);
        if (index < 0) continue;
        const Unit u = unit_at<kSplit>(p, index);
        if (u.n_tiles == 0) continue;
        const int n_tiles = u.n_tiles, part = u.part, m0 = u.m0, b = u.b;
        const int head = u.head0 + h;
        float m_used = -INFINITY, l = 0.f;

        for (int it = 0; it < n_tiles; ++it, ++tiles_done) {
            if ((n_tiles - 1 - it) % kStages == 0) ++terminal_uses;
            if (ok) ok = tc::mbar_wait(&bars->s_full[h], tiles_done & 1);  // after a failed wait: keep the barrier pattern, skip waits
            if (it == 0) TC_TRACE_EVENT(30);
            tc::tc_fence_after_sync();
            float s[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) tc::tmem_ld32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
            tc::tmem_wait_ld();
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&bars->s_free[h]);  // the score buffer may be overwritten by the other head
            if (it == 0 && part == 0) {
                // Diagonal tile: key column j is visible to query row i only if j <= i.
#pragma unroll
                for (int j = 0; j < 128; ++j) s[j] = j > row ? -INFINITY : s[j];
            }
            float mx[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) mx[q] = max3(s[q * 32], s[q * 32 + 1], s[q * 32 + 2]);
#pragma unroll
            for (int j = 3; j + 1 < 32; j += 2) {
#pragma unroll
                for (int q = 0; q < 4; ++q) mx[q] = max3(mx[q], s[q * 32 + j], s[q * 32 + j + 1]);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) mx[q] = fmaxf(mx[q], s[q * 32 + 31]);
            const float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            // Gated rescale: O and l are only brought to a new reference maximum when the row maximum
            // grew by more than 2^kRescaleThreshold, and only if some row of the warp needs it (the
            // TMEM accesses are warp-collective). The decision needs only the maxima; the rescale itself
            // waits for the previous tile's PV further down.
            float alpha = 1.f;
            bool rescale = false;
            if (it == 0) {
                m_used = tile_max;  // finite: column `row` of the diagonal tile is always visible, other tiles fully
            } else {
                const float m_new = fmaxf(m_used, tile_max);
                const bool grow = (m_new - m_used) * p.scale_log2 > kRescaleThreshold;
                rescale = __any_sync(0xffffffffu, grow);
                if (rescale) {
                    const float m_target = grow ? m_new : m_used;
                    alpha = tc::fast_exp2((m_used - m_target) * p.scale_log2);
                    m_used = m_target;
                }
            }
            const float neg_bias = -m_used * p.scale_log2;
            const float2 bias2 = make_float2(neg_bias, neg_bias);
            float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            // One chunk = 32 keys: x = s*scale - bias on packed pairs (fma.rn.f32x2), 2^x on the
            // exponential unit, packed row sums, BF16 pack for this head's P columns.
            auto chunk = [&](int c, uint32_t (&packed)[16]) {
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const float2 x = __ffma2_rn(make_float2(s[c * 32 + j], s[c * 32 + j + 1]), scale2, bias2);
                    const float2 e = make_float2(tc::fast_exp2(x.x), tc::fast_exp2(x.y));
                    sum2[(j >> 1) & 1] = __fadd2_rn(sum2[(j >> 1) & 1], e);
                    packed[j >> 1] = tc::pack_bf16x2(e.x, e.y);
                }
            };
            // PV of the previous tile reads P: its first half (keys 0-63, P chunks 0 and 1) must be done
            // before chunk 0 is rewritten, all of it before chunk 2 is rewritten or O is rescaled. Waiting
            // only for the first half here takes the second half's execution off this head's
            // exp -> PV -> exp chain; the full wait follows before chunk 2, by when it has long finished.
            // (The first tile of a unit follows an epilogue that has already waited for the previous unit's
            // last PV.)
            bool pv_done = it == 0;
            if (it > 0) {
                if (rescale) {
                    if (ok) ok = tc::mbar_wait(&bars->o_done[h], (tiles_done - 1) & 1);
                    pv_done = true;
                } else {
                    if (ok) ok = tc::mbar_wait(&bars->p_lo_free[h], (tiles_done - 1) & 1);
                }
                tc::tc_fence_after_sync();
                if (rescale) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t acc[32];
                        tc::tmem_ld32(o_tmem + c * 32, acc);
                        tc::tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[j] = __float_as_uint(__uint_as_float(acc[j]) * alpha);
                        tc::tmem_st32(o_tmem + c * 32, acc);
                    }
                    tc::tmem_wait_st();
                    l *= alpha;
                }
            }
            // The exponential unit is the scarcest resource, so the two heads take turns at it: while
            // one warpgroup exponentiates, the other head's P is being consumed by the tensor pipe
            // and its next S tile is produced. Head 0 goes first on every tile.
            if (h == 1 || tiles_done > 0) {
                // Hardware named barrier: the other warpgroup's 128 threads arrive without blocking when
                // their exponentials are issued, this warpgroup's 128 threads wait. It wakes faster than
                // an mbarrier wait; both sides execute it on every path so the counts always match.
                asm volatile("bar.sync %0, 256;" ::"r"(3 + h) : "memory");
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t packed[16];
                chunk(c, packed);
                // Hand the exponential unit over when this head's last exponentials are issued: the
                // other warpgroup needs about a hundred cycles to wake up.
                if (c == 3 && (h == 0 || tiles_done + 1 < cta_tiles))
                    asm volatile("bar.arrive %0, 256;" ::"r"(3 + (1 - h)) : "memory");
                if (c == 2) {
                    // Chunks 0 and 1 were stored a whole chunk of arithmetic ago, so this wait is short.
                    tc::tmem_wait_st();
                    tc::tc_fence_before_sync();
                    tc::mbar_arrive(&bars->p_half[h][0]);
                }
                if (c == 2 && !pv_done) {
                    if (ok) ok = tc::mbar_wait(&bars->o_done[h], (tiles_done - 1) & 1);
                    tc::tc_fence_after_sync();
                    pv_done = true;
                }
                tc::tmem_st16(p_tmem + c * 16, packed);
            }
            tc::tmem_wait_st();
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&bars->p_half[h][1]);
            l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
        }

        // ------------------------------------------------------------------ epilogue of the unit
        // (tiles_done now counts this unit's tiles as well.)
        TC_TRACE_EVENT(31);
        const float inv = l > 0.f ? 1.f / l : 0.f;
        float row_lse = l > 0.f ? fmaf(m_used, p.scale, logf(l)) : INFINITY;
        const int rows_here = min(kBlockM, p.tokens - m0);
        float* lse_out = p.lse + (int64_t(b) * p.q_heads + head) * p.tokens + m0;
        const bool bulk_lse = rows_here == kBlockM && (p.tokens & 3) == 0;
        float* lse_stage = reinterpret_cast<float*>(
            kHandoff ? smem + (h == 0 ? PREFILL_LSE_HEAD0_OFFSET_BYTES : PREFILL_LSE_HEAD1_OFFSET_BYTES)
                     : smem + kBarrierOffset + kBarrierBytes + h * 512);
        // The LSE array goes to the planner's region in the released terminal K stage (or to the dedicated
        // area), is published with one barrier of the head's warpgroup and leaves with one bulk store. Without
        // key splitting that happens here, before the last PV has even finished, so that the stage is free for the
        // next unit's keys as early as possible.
        auto store_lse = [&](bool writes) {
            // Both heads' last score MMAs have read the terminal stage once its "empty" phase completed.
            if (ok) ok = tc::mbar_wait(&bars->k_empty[0], (terminal_uses - 1) & 1);
            if (writes) lse_stage[row] = row_lse;
            tc::fence_proxy_async_smem();
            wg_barrier(h);
            if (row == 0) {
                if (writes && bulk_lse && !bars->abort) {
                    tc::bulk_store_1d(lse_out, lse_stage, kBlockM * 4);
                    tc::bulk_commit();
                    tc::bulk_wait_read_all();
                }
                tc::mbar_arrive(&bars->lse_drained);
            }
            if (writes && !bulk_lse && row < rows_here) lse_out[row] = row_lse;
        };
        if constexpr (!kSplit) store_lse(true);
        TC_TRACE_EVENT(32);

        if (ok) ok = tc::mbar_wait(&bars->o_done[h], (tiles_done - 1) & 1);
        TC_TRACE_EVENT(33);
        if (!ok) {
            atomicCAS(p.status, 0, 14 + h);
            bars->abort = 1;
        }
        tc::tc_fence_after_sync();
        float own_weight = inv;        // what this CTA's accumulator is multiplied by in the stored O
        float other_weight = 0.f;      // key-split, second finisher: weight of the other CTA's normalised O
        const float4* other_o = nullptr;
        bool stores = true;
        if constexpr (kSplit) {
            if (u.all_tiles >= 2) {
                const int unit = ((((u.m_block * p.batch + b) * p.kv_heads + u.kvh) * 2 + u.pair) * 2) + h;
                int32_t* claim = p.tickets + 2 * unit;
                int32_t* ready = claim + 1;
                float4* slot_o = p.part_o + size_t(unit) * (kBlockM * kDim / 4);
                float* slot_lse = p.part_lse + size_t(unit) * kBlockM;
                if (row == 0) bars->role[h] = atomicAdd(claim, 1);
                wg_barrier(h);
                if (bars->role[h] == 0) {
                    // First to finish this head: publish normalised O (coalesced: a warp's rows are
                    // consecutive float4s of one column group) and LSE, then raise the ready word.
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t acc[32];
                        tc::tmem_ld32(o_tmem + c * 32, acc);
                        tc::tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            slot_o[(c * 8 + i) * kBlockM + row] =
                                make_float4(__uint_as_float(acc[i * 4 + 0]) * inv, __uint_as_float(acc[i * 4 + 1]) * inv,
                                            __uint_as_float(acc[i * 4 + 2]) * inv, __uint_as_float(acc[i * 4 + 3]) * inv);
                    }
                    slot_lse[row] = row_lse;
                    __threadfence();
                    wg_barrier(h);
                    if (row == 0) tc::store_release_gpu(ready, 1);
                    stores = false;
                } else {
                    // Second: the first is past its key loop (it claimed), so this wait is short.
                    if (row == 0 && !tc::wait_word_gpu(ready, 1)) {
                        atomicCAS(p.status, 0, 16 + h);
                        bars->abort = 1;
                    }
                    wg_barrier(h);
                    const float other_lse = __ldcg(slot_lse + row);
                    const float top = fmaxf(row_lse, other_lse);
                    const float merged = top + logf(expf(row_lse - top) + expf(other_lse - top));
                    own_weight = inv * expf(row_lse - merged);
                    other_weight = expf(other_lse - merged);
                    row_lse = merged;
                    other_o = slot_o;
                }
            }
            store_lse(stores);
        }
        // O (BF16) is staged in the output staging buffer in the TMA store layout. The two heads use the buffer in
        // turn: head 0 of a unit after head 1 of the previous unit, head 1 after head 0 of the same unit.
        uint8_t* o_stage = smem + kOutStageOffset;
        if (h == 0) {
            if (units_done > 0 && ok) ok = tc::mbar_wait(&bars->stage_drained[1], (units_done - 1) & 1);
        } else {
            if (ok) ok = tc::mbar_wait(&bars->stage_drained[0], units_done & 1);
        }
        if (stores) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t acc[32];
            tc::tmem_ld32(o_tmem + c * 32, acc);
            tc::tmem_wait_ld();
            if (c == 3) {
                // The accumulator is in registers: the next unit's first PV may overwrite it.
                tc::tc_fence_before_sync();
                tc::mbar_arrive(&bars->o_free[h]);
            }
            float value[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) value[j] = __uint_as_float(acc[j]) * own_weight;
            if constexpr (kSplit) {
                if (other_o != nullptr) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 other = __ldcg(other_o + (c * 8 + i) * kBlockM + row);
                        value[i * 4 + 0] = fmaf(other.x, other_weight, value[i * 4 + 0]);
                        value[i * 4 + 1] = fmaf(other.y, other_weight, value[i * 4 + 1]);
                        value[i * 4 + 2] = fmaf(other.z, other_weight, value[i * 4 + 2]);
                        value[i * 4 + 3] = fmaf(other.w, other_weight, value[i * 4 + 3]);
                    }
                }
            }
            uint8_t* half = o_stage + (c >> 1) * kHalfBytes + row * 128;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 word;
                word.x = tc::pack_bf16x2(value[i * 8 + 0], value[i * 8 + 1]);
                word.y = tc::pack_bf16x2(value[i * 8 + 2], value[i * 8 + 3]);
                word.z = tc::pack_bf16x2(value[i * 8 + 4], value[i * 8 + 5]);
                word.w = tc::pack_bf16x2(value[i * 8 + 6], value[i * 8 + 7]);
                const int chunk = (c & 1) * 4 + i;
                *reinterpret_cast<uint4*>(half + ((chunk ^ (row & 7)) << 4)) = word;
            }
        }
        tc::fence_proxy_async_smem();
        wg_barrier(h);  // the whole tile is staged
        if (row == 0) {
            if (!bars->abort) {
                tc::tma_store_4d(&omap, o_stage, 0, head, m0, b);
                tc::tma_store_4d(&omap, o_stage + kHalfBytes, 64, head, m0, b);
                tc::bulk_commit();
                tc::bulk_wait_read_all();  // shared memory must outlive the stores' reads; the writes finish on their own
            }
            tc::mbar_arrive(&bars->stage_drained[h]);
        }
        } else {
            // (key split, first finisher) Nothing is staged, but the phases of both barriers advance all the same.
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&bars->o_free[h]);
            if (row == 0) tc::mbar_arrive(&bars->stage_drained[h]);
        }
        TC_TRACE_EVENT(34);
        ++units_done;
        }
    }

    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem, kTmemColumns);
    }
}

// =============================================================================== one CTA per unit
// The schedule for long units (more than 32 key tiles): the grid holds one CTA per unit and the hardware deals
// them to the SMs as they come free, longest first. The CTA's own Q tile doubles as the staging area of its output
// tile, so the arena ends behind the V ring.
constexpr int kRowblockBarrierOffset = kVOffset + kStages * kTileBytes;
constexpr int rowblock_shared_bytes(bool handoff) {
    return 1024 + kRowblockBarrierOffset + kBarrierBytes + (handoff ? 0 : kStagingBytes);
}

struct RowblockBarriers {
    uint64_t q_full;
    uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
    uint64_t s_full[2], s_free[2], p_half[2][2], p_lo_free[2], o_done[2];
    uint32_t tmem_base;
    int32_t abort;
    int32_t role[2];  // key-split only: which of the two CTAs of a query tile claimed each head first
};
static_assert(sizeof(RowblockBarriers) <= kBarrierBytes, "barrier block");

// kSplit: two CTAs per query tile, the first takes the key tiles nearest the diagonal (rounded up), the
// second the rest; whichever finishes a head second merges the other's normalised O and LSE into its own
// (LSE-weighted) and stores. For launches whose query tiles are too few to fill the GPU, where the longest
// tile alone would set the run time.
template <bool kHandoff, bool kSplit = false>
__global__ void __launch_bounds__(kThreads, 1)
prefill_rowblock_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
               const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap omap,
               const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    RowblockBarriers* bars = reinterpret_cast<RowblockBarriers*>(smem + kRowblockBarrierOffset);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Longest query tiles first; neighbouring CTAs share a KV head so K/V tiles hit in L2.
    const int per_block = p.batch * p.kv_heads * 2 * (kSplit ? 2 : 1);
    const int m_block = p.m_blocks - 1 - int(blockIdx.x) / per_block;
    int rest = int(blockIdx.x) % per_block;
    const int part = kSplit ? (rest & 1) : 0;
    if (kSplit) rest >>= 1;
    const int pair = rest & 1;
    const int kvh = (rest >> 1) % p.kv_heads;
    const int b = rest / (2 * p.kv_heads);
    const int head0 = kvh * kGroup + pair * 2;
    const int m0 = m_block * kBlockM;
    // Key tiles m_block, m_block-1, ..., 0; this CTA's share is n_tiles of them starting at key_block0.
    const int all_tiles = m_block + 1;
    const int near_tiles = kSplit ? (all_tiles + 1) / 2 : all_tiles;
    const int n_tiles = part == 0 ? near_tiles : all_tiles - near_tiles;
    const int key_block0 = part == 0 ? m_block : m_block - near_tiles;
    if (kSplit && n_tiles == 0) return;  // a one-tile row block has nothing to split

    // The TMA producer owns the operand barriers: it initialises them itself and sends for Q and for
    // the first ring stages at once, so the first loads are in flight while the other warps set up
    // their barriers and tensor memory. Everything else waits for the CTA barrier below.
    const uint64_t keep = tc::policy_evict_last(), stream_once = tc::policy_evict_first();
    auto load_kv = [&](int it) {
        const int stage = (n_tiles - 1 - it) % kStages;
        const int n0 = (key_block0 - it) * kBlockN;
        uint8_t* kdst = smem + kKOffset + stage * kTileBytes;
        tc::mbar_arrive_expect_tx(&bars->k_full[stage], kTileBytes);
        tc::tma_load_4d(kdst, &kmap, &bars->k_full[stage], 0, kvh, n0, b, keep);
        tc::tma_load_4d(kdst + kHalfBytes, &kmap, &bars->k_full[stage], 64, kvh, n0, b, keep);
        return stage;
    };
    auto load_v = [&](int it, int stage) {
        const int n0 = (key_block0 - it) * kBlockN;
        uint8_t* vdst = smem + kVOffset + stage * kTileBytes;
        tc::mbar_arrive_expect_tx(&bars->v_full[stage], kTileBytes);
        tc::tma_load_4d(vdst, &vmap, &bars->v_full[stage], 0, kvh, n0, b, keep);
        tc::tma_load_4d(vdst + kHalfBytes, &vmap, &bars->v_full[stage], 64, kvh, n0, b, keep);
    };
    if (threadIdx.x == kProducerWarp * 32) {
        tc::mbar_init(&bars->q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(&bars->k_full[s], 1);
            tc::mbar_init(&bars->k_empty[s], 2);  // one arrival per head's MMA issuer
            tc::mbar_init(&bars->v_full[s], 1);
            tc::mbar_init(&bars->v_empty[s], 2);
        }
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&qmap);
        tc::tma_prefetch_desc(&kmap);
        tc::tma_prefetch_desc(&vmap);
        tc::mbar_arrive_expect_tx(&bars->q_full, 2 * kTileBytes);
        for (int h = 0; h < 2; ++h) {
            uint8_t* dst = smem + kQOffset + h * kTileBytes;
            tc::tma_load_4d(dst, &qmap, &bars->q_full, 0, head0 + h, m0, b, stream_once);
            tc::tma_load_4d(dst + kHalfBytes, &qmap, &bars->q_full, 64, head0 + h, m0, b, stream_once);
        }
        for (int it = 0; it < kStages && it < n_tiles; ++it) load_v(it, load_kv(it));  // fresh stages: nothing to wait for
    }
    if (threadIdx.x == 0) {
        for (int h = 0; h < 2; ++h) {
            tc::mbar_init(&bars->s_full[h], 1);
            tc::mbar_init(&bars->s_free[h], kSoftmaxThreads);
            tc::mbar_init(&bars->p_half[h][0], kSoftmaxThreads);
            tc::mbar_init(&bars->p_half[h][1], kSoftmaxThreads);
            tc::mbar_init(&bars->o_done[h], 1);
            tc::mbar_init(&bars->p_lo_free[h], 1);
        }
        bars->abort = 0;
        tc::mbar_fence_init();
    }
    if (warp == kMmaWarp) {
        tc::tmem_alloc(&bars->tmem_base, kTmemColumns);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem = bars->tmem_base;

    // The third warpgroup only moves data and issues MMAs: it hands most of its registers to the
    // two softmax warpgroups, which keep a whole 128-column score row per thread. Each role's code
    // sits under its own setmaxnreg so that the register allocator sees the right budget.
    if (warp >= 2 * (kSoftmaxThreads / 32)) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kDataRegisters));
    if (warp == kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int it = kStages; it < n_tiles; ++it) {
                const int stage = (n_tiles - 1 - it) % kStages;
                const uint32_t parity = (uint32_t(it / kStages) & 1) ^ 1;
                if (!tc::mbar_wait(&bars->k_empty[stage], parity)) { atomicCAS(p.status, 0, 11); break; }
                load_kv(it);
                if (!tc::mbar_wait(&bars->v_empty[stage], parity)) { atomicCAS(p.status, 0, 12); break; }
                load_v(it, stage);
            }
        }
    } else {
        // ------------------------------------------------------------------ MMA issuers
        // Warp 9 issues every score MMA (the shared score buffer is used 0,1,0,1,... so their order is
        // fixed anyway); warps 10 and 11 issue PV for head 0 and head 1. Each role is one elected thread.
        // Issue blocks at the tensor pipe's rate and every barrier check costs such a lone thread
        // 100-170 cycles, so a thread that is busy issuing one kind of MMA must not be the one that has
        // to notice that the other kind has become ready.
        if (lane == 0) {
            constexpr uint32_t idesc_qk = tc::umma_idesc(128, 128, 1, 0, 0);
            constexpr uint32_t idesc_pv = tc::umma_idesc(128, 128, 1, 0, 1);
            auto stage_of = [&](int it) { return (n_tiles - 1 - it) % kStages; };
            auto parity_of = [&](int it) { return uint32_t(it / kStages) & 1; };
            bool ok = true;
            if (warp == kMmaWarp) {
                // S = Q_h K^T into the shared score buffer: both operands K-major, 8 steps of 16 along D
                // (4 per 64-element half). A score MMA may overwrite the buffer once the other head's
                // softmax warpgroup has pulled its tile into registers; because P has its own columns it
                // does not wait for any PV.
                const uint32_t q_addr = tc::smem_u32(smem + kQOffset);
                const uint32_t k_addr = tc::smem_u32(smem + kKOffset);
                ok = tc::mbar_wait(&bars->q_full, 0);
                for (int it = 0; ok && it < n_tiles; ++it) {
                    if (!(ok = tc::mbar_wait(&bars->k_full[stage_of(it)], parity_of(it)))) break;
                    const uint32_t kb = k_addr + stage_of(it) * kTileBytes;
                    for (int h = 0; h < 2 && ok; ++h) {
                        if (h == 0) {
                            if (it > 0) ok = tc::mbar_wait(&bars->s_free[1], uint32_t(it - 1) & 1);
                        } else {
                            ok = tc::mbar_wait(&bars->s_free[0], uint32_t(it) & 1);
                        }
                        if (!ok) break;
                        tc::tc_fence_after_sync();
#pragma unroll
                        for (int ks = 0; ks < 8; ++ks) {
                            const uint32_t off = uint32_t(ks >> 2) * kHalfBytes + uint32_t(ks & 3) * 32;
                            tc::umma_ss(tmem + s_column(h), tc::umma_desc_sw128(q_addr + h * kTileBytes + off, 16, 1024),
                                        tc::umma_desc_sw128(kb + off, 16, 1024), idesc_qk, ks > 0);
                        }
                        tc::umma_commit(&bars->s_full[h]);
                        tc::umma_commit(&bars->k_empty[stage_of(it)]);  // two arrivals per stage: one per head
                    }
                }
            } else {
                // O_h += P_h V, one 64-key half at a time: P from TMEM (8 columns per 16 keys), V MN-major
                // (row = key, 128 bytes per 64 d; the d halves 16 KiB apart, 8-key groups 1 KiB).
                const int h = warp - (kMmaWarp + 1);
                const uint32_t v_addr = tc::smem_u32(smem + kVOffset);
                const uint32_t p_col = tmem + p_column(h);
                const uint32_t o_col = tmem + o_column(h);
                auto issue_pv_half = [&](int it, int half) {
                    const uint32_t vb = v_addr + stage_of(it) * kTileBytes;
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const int ks = half * 4 + k4;
                        tc::umma_ts(o_col, p_col + uint32_t(ks) * 8, tc::umma_desc_sw128(vb + ks * 2048, kHalfBytes, 1024),
                                    idesc_pv, !(it == 0 && ks == 0));
                    }
                };
                for (int it = 0; ok && it < n_tiles; ++it) {
                    if (!(ok = tc::mbar_wait(&bars->v_full[stage_of(it)], parity_of(it)))) break;
                    if (!(ok = tc::mbar_wait(&bars->p_half[h][0], uint32_t(it) & 1))) break;
                    tc::tc_fence_after_sync();
                    issue_pv_half(it, 0);
                    tc::umma_commit(&bars->p_lo_free[h]);  // P columns of the first 64 keys may be rewritten
                    if (!(ok = tc::mbar_wait(&bars->p_half[h][1], uint32_t(it) & 1))) break;
                    tc::tc_fence_after_sync();
                    issue_pv_half(it, 1);
                    tc::umma_commit(&bars->o_done[h]);
                    tc::umma_commit(&bars->v_empty[stage_of(it)]);
                }
            }
            if (!ok) {
                atomicCAS(p.status, 0, 13);
                bars->abort = 1;
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegisters));
        // ------------------------------------------------------------------ softmax warpgroups
        const int h = warp >> 2;                        // head slot
        const int row = threadIdx.x & (kSoftmaxThreads - 1);
        const uint32_t lane_field = uint32_t((warp & 3) * 32) << 16;
        const uint32_t s_tmem = tmem + lane_field + s_column(h);
        const uint32_t p_tmem = tmem + lane_field + p_column(h);
        const uint32_t o_tmem = tmem + lane_field + o_column(h);
        const int head = head0 + h;
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;

        for (int it = 0; it < n_tiles; ++it) {
            if (ok) ok = tc::mbar_wait(&bars->s_full[h], uint32_t(it) & 1);  // after a failed wait: keep the barrier pattern, skip waits
            tc::tc_fence_after_sync();
            float s[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) tc::tmem_ld32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
            tc::tmem_wait_ld();
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&bars->s_free[h]);  // the score buffer may be overwritten by the other head
            if (it == 0 && part == 0) {
                // Diagonal tile: key column j is visible to query row i only if j <= i.
#pragma unroll
                for (int j = 0; j < 128; ++j) s[j] = j > row ? -INFINITY : s[j];
            }
            float mx[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) mx[q] = max3(s[q * 32], s[q * 32 + 1], s[q * 32 + 2]);
#pragma unroll
            for (int j = 3; j + 1 < 32; j += 2) {
#pragma unroll
                for (int q = 0; q < 4; ++q) mx[q] = max3(mx[q], s[q * 32 + j], s[q * 32 + j + 1]);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) mx[q] = fmaxf(mx[q], s[q * 32 + 31]);
            const float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            // Gated rescale: O and l are only brought to a new reference maximum when the row maximum
            // grew by more than 2^kRescaleThreshold, and only if some row of the warp needs it (the
            // TMEM accesses are warp-collective). The decision needs only the maxima; the rescale itself
            // waits for the previous tile's PV further down.
            float alpha = 1.f;
            bool rescale = false;
            if (it == 0) {
                m_used = tile_max;  // finite: column `row` of the diagonal tile is always visible, other tiles fully
            } else {
                const float m_new = fmaxf(m_used, tile_max);
                const bool grow = (m_new - m_used) * p.scale_log2 > kRescaleThreshold;
                rescale = __any_sync(0xffffffffu, grow);
                if (rescale) {
                    const float m_target = grow ? m_new : m_used;
                    alpha = tc::fast_exp2((m_used - m_target) * p.scale_log2);
                    m_used = m_target;
                }
            }
            const float neg_bias = -m_used * p.scale_log2;
            const float2 bias2 = make_float2(neg_bias, neg_bias);
            float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            // One chunk = 32 keys: x = s*scale - bias on packed pairs (fma.rn.f32x2), 2^x on the
            // exponential unit, packed row sums, BF16 pack for this head's P columns.
            auto chunk = [&](int c, uint32_t (&packed)[16]) {
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const float2 x = __ffma2_rn(make_float2(s[c * 32 + j], s[c * 32 + j + 1]), scale2, bias2);
                    const float2 e = make_float2(tc::fast_exp2(x.x), tc::fast_exp2(x.y));
                    sum2[(j >> 1) & 1] = __fadd2_rn(sum2[(j >> 1) & 1], e);
                    packed[j >> 1] = tc::pack_bf16x2(e.x, e.y);
                }
            };
            // PV of the previous tile reads P: its first half (keys 0-63, P chunks 0 and 1) must be done
            // before chunk 0 is rewritten, all of it before chunk 2 is rewritten or O is rescaled. Waiting
            // only for the first half here takes the second half's execution off this head's
            // exp -> PV -> exp chain; the full wait follows before chunk 2, by when it has long finished.
            bool pv_done = it == 0;
            if (it > 0) {
                if (rescale) {
                    if (ok) ok = tc::mbar_wait(&bars->o_done[h], uint32_t(it - 1) & 1);
                    pv_done = true;
                } else {
                    if (ok) ok = tc::mbar_wait(&bars->p_lo_free[h], uint32_t(it - 1) & 1);
                }
                tc::tc_fence_after_sync();
                if (rescale) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t acc[32];
                        tc::tmem_ld32(o_tmem + c * 32, acc);
                        tc::tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[j] = __float_as_uint(__uint_as_float(acc[j]) * alpha);
                        tc::tmem_st32(o_tmem + c * 32, acc);
                    }
                    tc::tmem_wait_st();
                    l *= alpha;
                }
            }
            // The exponential unit is the scarcest resource, so the two heads take turns at it: while
            // one warpgroup exponentiates, the other head's P is being consumed by the tensor pipe
            // and its next S tile is produced. Head 0 goes first on every tile.
            if (h == 1 || it > 0) {
                // Hardware named barrier: the other warpgroup's 128 threads arrive without blocking when
                // their exponentials are issued, this warpgroup's 128 threads wait. It wakes faster than
                // an mbarrier wait; both sides execute it on every path so the counts always match.
                asm volatile("bar.sync %0, 256;" ::"r"(3 + h) : "memory");
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t packed[16];
                chunk(c, packed);
                // Hand the exponential unit over when this head's last exponentials are issued: the
                // other warpgroup needs about a hundred cycles to wake up.
                if (c == 3 && (h == 0 || it + 1 < n_tiles))
                    asm volatile("bar.arrive %0, 256;" ::"r"(3 + (1 - h)) : "memory");
                if (c == 2) {
                    // Chunks 0 and 1 were stored a whole chunk of arithmetic ago, so this wait is short.
                    tc::tmem_wait_st();
                    tc::tc_fence_before_sync();
                    tc::mbar_arrive(&bars->p_half[h][0]);
                }
                if (c == 2 && !pv_done) {
                    if (ok) ok = tc::mbar_wait(&bars->o_done[h], uint32_t(it - 1) & 1);
                    tc::tc_fence_after_sync();
                    pv_done = true;
                }
                tc::tmem_st16(p_tmem + c * 16, packed);
            }
            tc::tmem_wait_st();
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&bars->p_half[h][1]);
            l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
        }

        // ------------------------------------------------------------------ epilogue
        if (ok) ok = tc::mbar_wait(&bars->o_done[h], uint32_t(n_tiles - 1) & 1);
        if (!ok) {
            atomicCAS(p.status, 0, 14 + h);
            bars->abort = 1;
        }
        tc::tc_fence_after_sync();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        float row_lse = l > 0.f ? fmaf(m_used, p.scale, logf(l)) : INFINITY;
        float own_weight = inv;        // what this CTA's accumulator is multiplied by in the stored O
        float other_weight = 0.f;      // key-split, second finisher: weight of the other CTA's normalised O
        const float4* other_o = nullptr;
        bool stores = true;
        if constexpr (kSplit) {
            if (all_tiles >= 2) {
                const int unit = ((((m_block * p.batch + b) * p.kv_heads + kvh) * 2 + pair) * 2) + h;
                int32_t* claim = p.tickets + 2 * unit;
                int32_t* ready = claim + 1;
                float4* slot_o = p.part_o + size_t(unit) * (kBlockM * kDim / 4);
                float* slot_lse = p.part_lse + size_t(unit) * kBlockM;
                if (row == 0) bars->role[h] = atomicAdd(claim, 1);
                wg_barrier(h);
                if (bars->role[h] == 0) {
                    // First to finish this head: publish normalised O (coalesced: a warp's rows are
                    // consecutive float4s of one column group) and LSE, then raise the ready word.
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t acc[32];
                        tc::tmem_ld32(o_tmem + c * 32, acc);
                        tc::tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            slot_o[(c * 8 + i) * kBlockM + row] =
                                make_float4(__uint_as_float(acc[i * 4 + 0]) * inv, __uint_as_float(acc[i * 4 + 1]) * inv,
                                            __uint_as_float(acc[i * 4 + 2]) * inv, __uint_as_float(acc[i * 4 + 3]) * inv);
                    }
                    slot_lse[row] = row_lse;
                    __threadfence();
                    wg_barrier(h);
                    if (row == 0) tc::store_release_gpu(ready, 1);
                    stores = false;
                } else {
                    // Second: the first is past its key loop (it claimed), so this wait is short.
                    if (row == 0 && !tc::wait_word_gpu(ready, 1)) {
                        atomicCAS(p.status, 0, 16 + h);
                        bars->abort = 1;
                    }
                    wg_barrier(h);
                    const float other_lse = __ldcg(slot_lse + row);
                    const float top = fmaxf(row_lse, other_lse);
                    const float merged = top + logf(expf(row_lse - top) + expf(other_lse - top));
                    own_weight = inv * expf(row_lse - merged);
                    other_weight = expf(other_lse - merged);
                    row_lse = merged;
                    other_o = slot_o;
                }
            }
        }
        if (stores) {
        // O (bf16) is staged over this head's own Q tile in the TMA store layout; LSE goes to the
        // planner's region in the released terminal K stage (or to the dedicated area).
        uint8_t* o_stage = smem + kQOffset + h * kTileBytes;
        float* lse_stage = reinterpret_cast<float*>(
            kHandoff ? smem + (h == 0 ? PREFILL_LSE_HEAD0_OFFSET_BYTES : PREFILL_LSE_HEAD1_OFFSET_BYTES)
                     : smem + kRowblockBarrierOffset + kBarrierBytes + h * 512);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t acc[32];
            tc::tmem_ld32(o_tmem + c * 32, acc);
            tc::tmem_wait_ld();
            float value[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) value[j] = __uint_as_float(acc[j]) * own_weight;
            if constexpr (kSplit) {
                if (other_o != nullptr) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 other = __ldcg(other_o + (c * 8 + i) * kBlockM + row);
                        value[i * 4 + 0] = fmaf(other.x, other_weight, value[i * 4 + 0]);
                        value[i * 4 + 1] = fmaf(other.y, other_weight, value[i * 4 + 1]);
                        value[i * 4 + 2] = fmaf(other.z, other_weight, value[i * 4 + 2]);
                        value[i * 4 + 3] = fmaf(other.w, other_weight, value[i * 4 + 3]);
                    }
                }
            }
            uint8_t* half = o_stage + (c >> 1) * kHalfBytes + row * 128;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 word;
                word.x = tc::pack_bf16x2(value[i * 8 + 0], value[i * 8 + 1]);
                word.y = tc::pack_bf16x2(value[i * 8 + 2], value[i * 8 + 3]);
                word.z = tc::pack_bf16x2(value[i * 8 + 4], value[i * 8 + 5]);
                word.w = tc::pack_bf16x2(value[i * 8 + 6], value[i * 8 + 7]);
                const int chunk = (c & 1) * 4 + i;
                *reinterpret_cast<uint4*>(half + ((chunk ^ (row & 7)) << 4)) = word;
            }
        }
        lse_stage[row] = row_lse;
        tc::fence_proxy_async_smem();
        wg_barrier(h);  // one barrier publishes the O tile and the LSE array of this head
        const int rows_here = min(kBlockM, p.tokens - m0);
        float* lse_out = p.lse + (int64_t(b) * p.q_heads + head) * p.tokens + m0;
        const bool bulk_lse = rows_here == kBlockM && (p.tokens & 3) == 0;
        if (row == 0 && !bars->abort) {
            tc::tma_store_4d(&omap, o_stage, 0, head, m0, b);
            tc::tma_store_4d(&omap, o_stage + kHalfBytes, 64, head, m0, b);
            if (bulk_lse) tc::bulk_store_1d(lse_out, lse_stage, kBlockM * 4);
            tc::bulk_commit();
            tc::bulk_wait_read_all();  // shared memory must outlive the stores' reads; the writes finish on their own
        }
        if (!bulk_lse && row < rows_here) lse_out[row] = row_lse;
        }
    }

    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem, kTmemColumns);
    }
}

// ------------------------------------------------------------------------------- host side
int check_geometry(int device, int64_t batch, int64_t tokens, int64_t q_heads, int64_t num_splits, int64_t mapping,
                   int causal, tc::DeviceInfo* info) {
    int status = tc::require_sm100(device, info);
    if (status != TC_OK) return status;
    TC_REQUIRE(num_splits == 0 && (mapping == 0 || mapping == 1), "prefill requires num_splits=0 and mapping 0 or 1");
    TC_REQUIRE(causal, "Full causal no-past prefill requires causal=True");
    TC_REQUIRE(q_heads >= 4 && q_heads <= 32 && q_heads % 4 == 0, "Q must be [B,T,Hq,128] with Hq a multiple of 4 up to 32");
    TC_REQUIRE(batch == 1 || batch == 4, "The shared-LSE schedule requires batch 1 or 4");
    TC_REQUIRE(tokens >= 128 && tokens <= 32768, "The shared-LSE schedule requires 128-32768 tokens");
    TC_REQUIRE(info->smem_optin >= shared_bytes(false), "device lacks the opt-in shared memory this schedule needs");
    return TC_OK;
}

int check_strides(const char* name, const int64_t strides[3], int64_t batch, int64_t tokens, int64_t heads) {
    TC_REQUIRE(strides, "null strides");
    const int64_t sizes[3] = {batch, tokens, heads};
    for (int axis = 0; axis < 3; ++axis) {
        TC_REQUIRE(strides[axis] >= 0, "%s: negative strides are outside this ABI", name);
        if (sizes[axis] > 1)
            TC_REQUIRE(strides[axis] % 8 == 0 && strides[axis] >= 128,
                       "%s: strides must be multiples of 8 elements with a contiguous last dimension", name);
    }
    return TC_OK;
}

size_t span_bytes(const int64_t strides[3], int64_t batch, int64_t tokens, int64_t heads) {
    return size_t((batch - 1) * strides[0] + (tokens - 1) * strides[1] + (heads - 1) * strides[2] + kDim) * 2;
}

// Key-split workspace: [claim, ready] words per unit (a unit is one head of one query tile), padded to 256
// bytes, then the units' 64 KiB O slots, then their 512-byte LSE slots.
struct SplitLayout {
    int64_t units, ticket_bytes, o_offset, lse_offset, total;
};
SplitLayout split_layout(int64_t batch, int64_t tokens, int64_t q_heads) {
    SplitLayout w;
    w.units = ((tokens + kBlockM - 1) / kBlockM) * batch * q_heads;
    w.ticket_bytes = (w.units * 8 + 255) / 256 * 256;
    w.o_offset = w.ticket_bytes;
    w.lse_offset = w.o_offset + w.units * int64_t(kBlockM) * kDim * 4;
    w.total = w.lse_offset + w.units * int64_t(kBlockM) * 4;
    return w;
}

// Two CTAs per query tile pay off when the longest tile alone (m_blocks key tiles) would outlast an even
// share of all tiles per SM by a quarter or more, i.e. when the grid is too small to hide it, and the tiles
// are long enough (16 key tiles) to carry a second CTA's fixed cost and the merge. Measured on 148 SMs at
// 8192 tokens: 4 query heads 109 -> 71 us with two CTAs per tile, 8 heads 111 -> 133 us (not chosen).
bool split_pays_off(const tc::DeviceInfo& info, int64_t batch, int64_t tokens, int64_t q_heads) {
    const int64_t m_blocks = (tokens + kBlockM - 1) / kBlockM;
    const int64_t tile_pairs = batch * (q_heads / 2) * m_blocks * (m_blocks + 1) / 2;
    return m_blocks >= 16 && m_blocks * int64_t(info.sms) * 4 > tile_pairs * 5;
}

// Short units (up to 32 key tiles, i.e. 4096 tokens) go to one persistent CTA per SM, which saves a CTA's start-up
// per unit: 13 % at batch 4 x 2048 tokens, 3 % at batch 1 x 2048. Long units go to the schedule with one CTA per
// unit: the hardware's own dealing balances the SMs better than the fixed deal, and a change of unit inside a
// persistent CTA costs about as much as a new CTA (measured: the persistent schedule 4-8 % slower at 8192 tokens).
bool persistent_schedule(const PrefillParams& p) { return p.m_blocks <= 32; }

template <bool kHandoff, bool kSplit>
int launch(const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap, const CUtensorMap& omap,
           const PrefillParams& p, int sms, cudaStream_t stream) {
    static thread_local int configured_device = -1;
    int device = 0;
    TC_CUDA(cudaGetDevice(&device));
    if (configured_device != device) {
        TC_CUDA(cudaFuncSetAttribute(&prefill_kernel<kHandoff, kSplit>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     shared_bytes(kHandoff)));
        TC_CUDA(cudaFuncSetAttribute(&prefill_rowblock_kernel<kHandoff, kSplit>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     rowblock_shared_bytes(kHandoff)));
        configured_device = device;
    }
    // Either way the shared memory and the tensor memory of a CTA leave room for one CTA per SM.
    if (persistent_schedule(p)) {
        const unsigned grid = unsigned(p.total_units > sms ? sms : p.total_units);
        prefill_kernel<kHandoff, kSplit><<<grid, kThreads, shared_bytes(kHandoff), stream>>>(qmap, kmap, vmap, omap, p);
    } else {
        prefill_rowblock_kernel<kHandoff, kSplit>
            <<<unsigned(p.total_units), kThreads, rowblock_shared_bytes(kHandoff), stream>>>(qmap, kmap, vmap, omap, p);
    }
    TC_CUDA(cudaGetLastError());
    return TC_OK;
}

int prefill_common(int device, void* stream, const void* q, const int64_t q_strides[3], const void* k,
                   const int64_t k_strides[3], const void* v, const int64_t v_strides[3], void* out, float* lse,
                   int64_t batch, int64_t tokens, int64_t q_heads, int64_t num_splits, int64_t mapping, double scale,
                   int causal, void* workspace, int64_t workspace_bytes, int key_splits,
                   int64_t* key_splits_used = nullptr);

}  // namespace

extern "C" {

#ifdef TC_TRACE
// Trace builds only: copy out / clear the role logs of all CTAs (both synchronise the device).
int tc_debug_prefill_trace(void* host) {
    return cudaMemcpyFromSymbol(host, g_prefill_trace, sizeof(g_prefill_trace)) == cudaSuccess ? 0 : 1;
}
int tc_debug_prefill_trace_clear(void) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_prefill_trace) != cudaSuccess) return 1;
    return cudaMemset(address, 0, sizeof(g_prefill_trace)) == cudaSuccess ? 0 : 1;
}
#endif

int tc_prefill_workspace_spec(int device, int64_t batch, int64_t tokens, int64_t q_heads, int64_t num_splits,
                              int64_t mapping, int causal, int64_t spec[3]) {
    tc::DeviceInfo info;
    int status = check_geometry(device, batch, tokens, q_heads, num_splits, mapping, causal, &info);
    if (status != TC_OK) return status;
    TC_REQUIRE(spec, "null spec");
    spec[0] = 1;
    spec[1] = 0;
    spec[2] = 0;
    return TC_OK;
}

int tc_prefill_forward_out(int device, void* stream, const void* q, const int64_t q_strides[3], const void* k,
                           const int64_t k_strides[3], const void* v, const int64_t v_strides[3], void* out,
                           float* lse, int64_t workspace_o_elems, int64_t workspace_lse_elems, int64_t batch,
                           int64_t tokens, int64_t q_heads, int64_t num_splits, int64_t mapping, double scale,
                           int causal) {
    TC_REQUIRE(workspace_o_elems == 0 && workspace_lse_elems == 0, "Generated long prefill uses no split workspace");
    return prefill_common(device, stream, q, q_strides, k, k_strides, v, v_strides, out, lse, batch, tokens, q_heads,
                          num_splits, mapping, scale, causal, nullptr, 0, 1);
}

int tc_prefill_key_split_workspace_bytes(int64_t batch, int64_t tokens, int64_t q_heads, int64_t* bytes) {
    TC_REQUIRE(bytes && batch >= 1 && tokens >= 1 && q_heads >= 4 && q_heads % 4 == 0, "invalid geometry");
    *bytes = split_layout(batch, tokens, q_heads).total;
    return TC_OK;
}

int tc_prefill_key_split_forward_out(int device, void* stream, const void* q, const int64_t q_strides[3], const void* k,
                                     const int64_t k_strides[3], const void* v, const int64_t v_strides[3], void* out,
                                     float* lse, void* workspace, int64_t workspace_bytes, int64_t batch,
                                     int64_t tokens, int64_t q_heads, int64_t mapping, double scale, int64_t key_splits,
                                     int64_t* key_splits_used) {
    TC_REQUIRE(key_splits >= 0 && key_splits <= 2, "key_splits must be 0 (choose), 1 or 2");
    return prefill_common(device, stream, q, q_strides, k, k_strides, v, v_strides, out, lse, batch, tokens, q_heads, 0,
                          mapping, scale, 1, workspace, workspace_bytes, int(key_splits), key_splits_used);
}

}  // extern "C"

namespace {

int prefill_common(int device, void* stream, const void* q, const int64_t q_strides[3], const void* k,
                   const int64_t k_strides[3], const void* v, const int64_t v_strides[3], void* out, float* lse,
                   int64_t batch, int64_t tokens, int64_t q_heads, int64_t num_splits, int64_t mapping, double scale,
                   int causal, void* workspace, int64_t workspace_bytes, int key_splits, int64_t* key_splits_used) {
    tc::DeviceInfo info;
    int status = check_geometry(device, batch, tokens, q_heads, num_splits, mapping, causal, &info);
    if (status != TC_OK) return status;
    const int64_t kv_heads = q_heads / kGroup;
    TC_REQUIRE(q && k && v && out && lse, "null tensor pointer");
    if (key_splits == 0) key_splits = split_pays_off(info, batch, tokens, q_heads) ? 2 : 1;
    if (key_splits_used) *key_splits_used = key_splits;
    const SplitLayout split = split_layout(batch, tokens, q_heads);
    if (key_splits == 2) {
        TC_REQUIRE(workspace && reinterpret_cast<uintptr_t>(workspace) % 256 == 0 && workspace_bytes >= split.total,
                   "key-split prefill needs a 256-byte aligned workspace of tc_prefill_key_split_workspace_bytes bytes");
    }
    TC_REQUIRE(std::isfinite(scale) && scale > 0, "Finite positive model attention scale required");
    if ((status = check_strides("q", q_strides, batch, tokens, q_heads)) != TC_OK) return status;
    if ((status = check_strides("k", k_strides, batch, tokens, kv_heads)) != TC_OK) return status;
    if ((status = check_strides("v", v_strides, batch, tokens, kv_heads)) != TC_OK) return status;
    for (const void* pointer : {q, k, v, static_cast<const void*>(out)})
        TC_REQUIRE(reinterpret_cast<uintptr_t>(pointer) % 16 == 0, "Aligned native Q/K/V/O base required");
    TC_REQUIRE(reinterpret_cast<uintptr_t>(lse) % 16 == 0, "Aligned LSE base required");
    const size_t out_bytes = size_t(batch) * tokens * q_heads * kDim * 2, lse_bytes = size_t(batch) * q_heads * tokens * 4;
    const void* inputs[3] = {q, k, v};
    const size_t input_bytes[3] = {span_bytes(q_strides, batch, tokens, q_heads), span_bytes(k_strides, batch, tokens, kv_heads),
                                   span_bytes(v_strides, batch, tokens, kv_heads)};
    for (int i = 0; i < 3; ++i)
        TC_REQUIRE(!tc::ranges_overlap(out, out_bytes, inputs[i], input_bytes[i]) &&
                       !tc::ranges_overlap(lse, lse_bytes, inputs[i], input_bytes[i]),
                   "Writable output aliases actual strided input storage span");
    TC_REQUIRE(!tc::ranges_overlap(out, out_bytes, lse, lse_bytes), "O/LSE overlap");

    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    tc::DeviceScratch scratch;
    if ((status = tc::device_scratch(device, &scratch)) != TC_OK) return status;
    CUtensorMap qmap, kmap, vmap, omap;
    if ((status = tc::make_rows_map(&qmap, q, false, q_heads, tokens, batch, q_strides[2], q_strides[1], q_strides[0], kBlockM, 2)) != TC_OK) return status;
    if ((status = tc::make_rows_map(&kmap, k, false, kv_heads, tokens, batch, k_strides[2], k_strides[1], k_strides[0], kBlockN, 2)) != TC_OK) return status;
    if ((status = tc::make_rows_map(&vmap, v, false, kv_heads, tokens, batch, v_strides[2], v_strides[1], v_strides[0], kBlockN, 2)) != TC_OK) return status;
    if ((status = tc::make_rows_map(&omap, out, false, q_heads, tokens, batch, kDim, q_heads * kDim, tokens * q_heads * kDim, kBlockM, 2)) != TC_OK) return status;

    PrefillParams p{};
    p.lse = lse;
    p.status = scratch.status;
    p.batch = int(batch);
    p.tokens = int(tokens);
    p.q_heads = int(q_heads);
    p.kv_heads = int(kv_heads);
    p.m_blocks = int((tokens + kBlockM - 1) / kBlockM);
    p.total_units = p.m_blocks * p.batch * p.kv_heads * 2;
    p.scale = float(scale);
    p.scale_log2 = float(scale) * float(M_LOG2E);
    TC_REQUIRE(std::isfinite(p.scale_log2) && p.scale > 0.f, "attention scale is not a positive finite FP32 value");
    cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
    if (key_splits == 2) {
        uint8_t* base = static_cast<uint8_t*>(workspace);
        const void* tensors[5] = {q, k, v, out, lse};
        const size_t tensor_bytes[5] = {input_bytes[0], input_bytes[1], input_bytes[2], out_bytes, lse_bytes};
        for (int i = 0; i < 5; ++i)
            TC_REQUIRE(!tc::ranges_overlap(workspace, size_t(split.total), tensors[i], tensor_bytes[i]),
                       "workspace aliases a tensor");
        p.tickets = reinterpret_cast<int32_t*>(base);
        p.part_o = reinterpret_cast<float4*>(base + split.o_offset);
        p.part_lse = reinterpret_cast<float*>(base + split.lse_offset);
        TC_CUDA(cudaMemsetAsync(base, 0, size_t(split.ticket_bytes), cuda_stream));
        p.total_units *= 2;
        return mapping == 1 ? launch<true, true>(qmap, kmap, vmap, omap, p, info.sms, cuda_stream)
                            : launch<false, true>(qmap, kmap, vmap, omap, p, info.sms, cuda_stream);
    }
    return mapping == 1 ? launch<true, false>(qmap, kmap, vmap, omap, p, info.sms, cuda_stream)
                        : launch<false, false>(qmap, kmap, vmap, omap, p, info.sms, cuda_stream);
}

}  // namespace

extern "C" {

int tc_prefill_resources(int device, const int64_t q_strides[3], const int64_t k_strides[3],
                         const int64_t v_strides[3], int64_t batch, int64_t tokens, int64_t q_heads,
                         int64_t num_splits, int64_t mapping, int causal, int64_t* values, int64_t capacity,
                         int64_t* count) {
    tc::DeviceInfo info;
    int status = check_geometry(device, batch, tokens, q_heads, num_splits, mapping, causal, &info);
    if (status != TC_OK) return status;
    TC_REQUIRE(q_strides && k_strides && v_strides && values && count && capacity >= 46, "resources needs room for 46 values");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    const int64_t tiles = (tokens + kBlockM - 1) / kBlockM;
    const int64_t header[12] = {1, tokens, q_heads, kGroup, 1, batch * (q_heads / 2) * tiles, 0, 0, 0, kBlockM, kBlockN, 1};
    for (int i = 0; i < 12; ++i) values[i] = header[i];
    if (tiles <= 32)
        status = mapping == 1 ? tc::kernel_resources(&prefill_kernel<true>, kThreads, shared_bytes(true), values + 12)
                              : tc::kernel_resources(&prefill_kernel<false>, kThreads, shared_bytes(false), values + 12);
    else
        status = mapping == 1
                     ? tc::kernel_resources(&prefill_rowblock_kernel<true>, kThreads, rowblock_shared_bytes(true), values + 12)
                     : tc::kernel_resources(&prefill_rowblock_kernel<false>, kThreads, rowblock_shared_bytes(false), values + 12);
    if (status != TC_OK) return status;
    for (int i = 20; i < 28; ++i) values[i] = 0;
    const int64_t layout[18] = {0, tokens, tokens, q_heads, q_heads / kGroup, 1, MODEL_FAMILY_CODE,
                                q_strides[0], q_strides[1], q_strides[2], k_strides[0], k_strides[1], k_strides[2],
                                v_strides[0], v_strides[1], v_strides[2], q_strides[1], q_strides[2]};
    for (int i = 0; i < 18; ++i) values[28 + i] = layout[i];
    *count = 46;
    return TC_OK;
}

}  // extern "C"
