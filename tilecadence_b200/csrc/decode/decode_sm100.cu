// Split-KV decode for one query token per sequence (GQA, four query heads per KV head, D = 128)
// with the KV-cache append and the LSE-weighted split reduction fused into one launch.
//
// Path replaced: tilecadence/cuda/decode/decode.cu:158-193 (host checks and dispatch),
// ab_fused_splitkv.cuh:6-471 (split kernel, fused append :189-212, compact epilogue :327-397) and
// the separate combine launch (decode.cu:131-140).
//
// The kernel is HBM-bound: every visible K and V row is read exactly once, 256 bytes per row per
// KV head. One CTA = (batch, KV head, split). A producer warp streams 64-key K/V tiles through a
// ring of shared-memory stages with TMA (128-byte swizzle) and mbarriers; the four warps of a consumer
// group each own 16 keys of a tile and run QK^T / PV on warp-level bf16 MMAs with an online softmax, and
// two such groups take the tiles in turn, so arithmetic does not limit the stream even when the tiles
// come from L2. Split ranges follow the device-side lengths. The per-warp
// partials are merged through the released terminal stage: the four output rows and their LSE
// are staged at the planner's offsets inside the terminal V region, published with one barrier and
// exported with one 16-byte vector per thread. The last CTA to finish a (batch, KV head) merges
// the split partials, so no second launch is needed.
//
// Options on the same kernel: caches addressed through a block table (pages) or a per-sequence
// batch index (ab_fused_splitkv.cuh:92-103); rotary position embedding of q and of the appended K
// row applied in registers; a KV-sequence shard of a longer cache (global lengths, shard start)
// that writes a partial result; and, for shards spread over the GPUs of one node, the cross-GPU
// merge of those partials inside the launch through peer stores (template parameter kPeer).
#include "config.cuh"
#include "tc_host.cuh"
#include "tc_ptx.cuh"

#include <cmath>
#include <cstring>

namespace {

constexpr int kTileN = AB_DECODE_BLOCK_N;
constexpr int kStages = AB_DECODE_STAGES;
constexpr int kStageBytes = AB_DECODE_STAGE_BYTES;
constexpr int kHalfBytes = kTileN * 128;  // one 64-element half of the head dimension, all tile rows
constexpr int kVBytes = 2 * kHalfBytes;
constexpr int kGroupWarps = AB_DECODE_WARPS;        // warps that share one tile, 16 keys each
constexpr int kGroups = AB_DECODE_WARP_GROUPS;      // consumer groups that take the tiles in turn
constexpr int kConsumerWarps = kGroupWarps * kGroups;
constexpr int kConsumerThreads = 32 * kConsumerWarps;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kMergeThreads = 128;                  // four output rows x 32 lanes run the CTA's epilogue
// Tile `it` of a CTA's n tiles uses stage (n-1-it) % kStages and belongs to group (n-1-it) % kGroups, so the
// same (stage, group) pair comes round every kRingPeriod tiles. Each pair has a "full" barrier of its own: a
// group then sees every phase of the barriers it waits on, in order, and a parity wait can never mistake
// the other group's tile in that stage for its own.
constexpr int ring_period(int a, int b) {
    int x = a, y = b;
    while (y) { const int t = x % y; x = y; y = t; }
    return a / x * b;
}
constexpr int kRingPeriod = ring_period(kStages, kGroups);
// Registers per thread such that AB_DECODE_CTAS_PER_SM CTAs fit the 64 K registers of an SM (allocated per warp
// in multiples of 8 per thread).
constexpr int kMaxRegisters = 65536 / (AB_DECODE_CTAS_PER_SM * kThreads) / 8 * 8;
constexpr int kGroup = 4;  // query heads per KV head
constexpr int kDim = 128;
constexpr int kMaxSplits = 128;
constexpr int kPrefetchTiles = 12;  // tiles a CTA may prefetch into L2 beyond its shared-memory ring
constexpr int kEarlyLimitTiles = 32;  // shares longer than this stream nothing ahead of the stream dependency
constexpr int kStagingBytes = 2304;  // dedicated O/LSE staging when the handoff is disabled
constexpr int kBarrierBytes = 256;
// Cross-GPU exchange of per-rank partials (KV sequence sharded over the ranks of one node). Every
// rank owns one exchange block that all ranks map; its layout for `world` ranks and `units` =
// batch * KV heads is
//   slots  [2 epoch parities][world source ranks][units] x kPeerSlotBytes
//          flag-in-data words: thread t of the unit's 128 writes 32 bytes at t*32
//          {o.x, epoch, o.y, epoch, o.z, epoch, o.w, epoch}; the four partial LSE follow at 4096 + row*8
//          as {lse, epoch}
//   epochs [units] u32   calls completed by the owner (owner-private)
constexpr int kMaxPeers = 8;
constexpr int kPeerLseOffset = kGroup * kDim * 8;
constexpr int kPeerSlotBytes = kPeerLseOffset + 64;
__host__ __device__ constexpr size_t peer_epochs_offset(int world, int units) {
    return size_t(2) * world * units * kPeerSlotBytes;
}
__host__ __device__ constexpr size_t peer_block_bytes(int world, int units) {
    return (peer_epochs_offset(world, units) + size_t(units) * 4 + 255) / 256 * 256;
}

static_assert(kStageBytes == 2 * kVBytes, "a stage holds one V tile followed by one K tile");
static_assert(kMaxSplits % 32 == 0 && kGroup * kMaxSplits * 4 <= kVBytes, "split weights fit the terminal K stage");
static_assert(kTileN == 16 * kGroupWarps, "each warp of a consumer group owns 16 keys of a tile");
static_assert(kGroups >= 1 && kGroups <= kStages, "every consumer group parks its partial in a stage of its own");
static_assert(kMergeThreads <= kConsumerThreads && kMergeThreads == 32 * kGroupWarps, "epilogue threads");
static_assert(AB_DECODE_TERMINAL_V_BYTES == kVBytes, "planner donor size must match the V tile");
static_assert(AB_DECODE_O_OFFSET_BYTES % 16 == 0 && AB_DECODE_LSE_OFFSET_BYTES % 16 == 0, "vector export");
static_assert(AB_DECODE_O_OFFSET_BYTES + 2048 <= kVBytes && AB_DECODE_LSE_OFFSET_BYTES + 16 <= kVBytes,
              "handoff regions must lie inside the terminal V stage");
static_assert(AB_DECODE_O_OFFSET_BYTES + 2048 <= AB_DECODE_LSE_OFFSET_BYTES ||
                  AB_DECODE_LSE_OFFSET_BYTES + 16 <= AB_DECODE_O_OFFSET_BYTES,
              "handoff regions must not overlap");

constexpr int shared_bytes(bool handoff) {
    return 1024 + kStages * kStageBytes + kBarrierBytes + (handoff ? 0 : kStagingBytes);
}

struct DecodeParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* kcache;
    __nv_bfloat16* vcache;
    const __nv_bfloat16* knew;
    const __nv_bfloat16* vnew;
    const int32_t* old_lengths;
    __nv_bfloat16* out;  // final O, bf16 [B,1,Hq,128] (partial == 0)
    float* lse;          // final LSE [B,Hq] or partial LSE
    float* partial_o;    // fp32 [B,Hq,128] (partial == 1)
    float* ws_o;
    float* ws_lse;
    int32_t* tickets;
    int32_t* status;
    int batch, capacity, kv_heads, splits, append, partial;
    int64_t shard_start;
    float scale, scale_log2;
    uint8_t* peer_blocks[kMaxPeers];  // partial == 2: every rank's exchange block as mapped here
    int world, rank;
    // Indexed caches (ab_fused_splitkv.cuh:92-103). block_table != nullptr: the caches are pages
    // [cache_slots, page_size, Hkv, 128] and row r of sequence b lives in page
    // block_table[b * table_stride + r / page_size]; `capacity` is then pages_per_seq * page_size.
    // Otherwise cache_batch_idx (if set) picks the cache slot of sequence b and page_size == capacity.
    const int32_t* block_table;
    const int32_t* cache_batch_idx;
    int64_t table_stride;
    int page_size, cache_slots;
    // Rotary position embedding applied in the kernel to q and to the appended K row (both arrive
    // un-rotated): fp32 tables [rope_positions, 64], row = the token's position old_lengths[b].
    const float* rope_cos;
    const float* rope_sin;
    int rope_positions;
    // Caller's promise about the kernel launched just before this one on the stream. 1: it writes neither the
    // caches' visible rows, nor old_lengths, nor the index tables; 2: the same, except that it may have written
    // row old_lengths[b] - 1 of these caches (the previous decode step of the same sequences). The K/V stream
    // of the rows that are promised stable then starts before the stream dependency resolves.
    int cache_stable;
};

// Rotate-half RoPE of one (x[i], x[i + 64]) pair, i < 64, with every product and sum rounded to fp32
// on its own (no fused multiply-add), so that a host restatement gets the same bits:
//   lo' = x_lo * cos - x_hi * sin,   hi' = x_hi * cos + x_lo * sin.
__device__ __forceinline__ void rope_pair(float x_lo, float x_hi, float c, float sn, float& lo, float& hi) {
    lo = __fsub_rn(__fmul_rn(x_lo, c), __fmul_rn(x_hi, sn));
    hi = __fadd_rn(__fmul_rn(x_hi, c), __fmul_rn(x_lo, sn));
}
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }


// Cache slot (page, or batch entry of the cache tensor) and row inside it for logical row `row`.
__device__ __forceinline__ void locate_row(const DecodeParams& p, int b, int slot_of_b, int row, int& slot, int& local) {
    if (p.block_table) {
        const int page = row / p.page_size;
        int id = __ldg(p.block_table + int64_t(b) * p.table_stride + page);
        id = id < 0 ? 0 : (id >= p.cache_slots ? p.cache_slots - 1 : id);  // never leave the allocation
        slot = id;
        local = row - page * p.page_size;
    } else {
        slot = slot_of_b;
        local = row;
    }
}

__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }
__device__ __forceinline__ void merge_barrier() { asm volatile("bar.sync 2, %0;" ::"n"(kMergeThreads) : "memory"); }

__device__ __forceinline__ uint32_t swizzled(uint32_t row, uint32_t chunk16) {
    // Byte offset of 16-byte chunk `chunk16` (0..15 across the 128-element row) of tile row `row`
    // inside a K or V tile: two 64-element halves, each row 128 bytes, 128-byte TMA swizzle.
    return (chunk16 >> 3) * kHalfBytes + row * 128 + (((chunk16 & 7) ^ (row & 7)) << 4);
}

// LSE-weighted merge of `parts` normalised partial results for one output row (four columns per
// thread): LSE = ln sum_s e^{LSE_s}, O = sum_s e^{LSE_s - LSE} O_s. A part that saw no key has
// LSE = -inf and may hold anything: it is never multiplied. A row nobody saw gets O = 0, LSE = +inf.
// Both the standalone combine kernel and the in-launch cross-GPU merge use this one function, so
// the two routes give identical bits.
// kUnroll > 0 visits parts 0..kUnroll-1 with static indices (for operands held in registers) and
// skips those >= parts; the arithmetic, spelled with explicit roundings, is the same either way.
template <int kUnroll, class LoadLse, class LoadO>
__device__ __forceinline__ void lse_weighted_merge(int parts, LoadLse load_lse, LoadO load_o, float4& o, float& lse) {
    float lse_max = -INFINITY;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float total = 0.f;
    auto add = [&](int s) {
        const float part_lse = load_lse(s);
        const float4 v = load_o(s);
        if (part_lse != -INFINITY) {
            const float weight = __expf(__fsub_rn(part_lse, lse_max));
            total = __fadd_rn(total, weight);
            acc.x = __fmaf_rn(weight, v.x, acc.x);
            acc.y = __fmaf_rn(weight, v.y, acc.y);
            acc.z = __fmaf_rn(weight, v.z, acc.z);
            acc.w = __fmaf_rn(weight, v.w, acc.w);
        }
    };
    if constexpr (kUnroll > 0) {
#pragma unroll
        for (int s = 0; s < kUnroll; ++s)
            if (s < parts) lse_max = fmaxf(lse_max, load_lse(s));
        if (lse_max != -INFINITY) {
#pragma unroll
            for (int s = 0; s < kUnroll; ++s)
                if (s < parts) add(s);
        }
    } else {
        for (int s = 0; s < parts; ++s) lse_max = fmaxf(lse_max, load_lse(s));
        if (lse_max != -INFINITY)
            for (int s = 0; s < parts; ++s) add(s);
    }
    const float inv = total > 0.f ? __frcp_rn(total) : 0.f;
    o = make_float4(__fmul_rn(acc.x, inv), __fmul_rn(acc.y, inv), __fmul_rn(acc.z, inv), __fmul_rn(acc.w, inv));
    lse = total > 0.f ? __fadd_rn(lse_max, logf(total)) : INFINITY;
}

// Build switch TC_TRACE (off in every shipped library): thread 0 and the producer's lane 0 of every CTA
// record %globaltimer at the points named below into a device table that tc_debug_trace copies out. It is how
// the time-line tables of a decode step are made; see tilecadence_b200/trace_decode.py.
//   0 entry  1 CTA sequence number  2 split | kv head << 8 | tiles << 16  3 lengths known, barriers ready
//   4+2t / 5+2t tile t arrived / consumed (t < 8)  20 key loop done  21 partial staged  22 ticket taken
//   19 result stored  23 SM id  24 (producer) first ring tiles issued  25 prefetches issued  26 last tile issued
//   27 stream dependency resolved (consumers)  28 last CTA of a head: split LSEs loaded  29 split partials merged
#ifdef TC_TRACE
__device__ unsigned long long g_trace[1024][32];
__device__ unsigned int g_trace_ctas;
#define TC_TRACE_POINT(slot) do { if (trace_row) trace_row[slot] = tc::global_timer_ns(); } while (0)
#else
#define TC_TRACE_POINT(slot) do { } while (0)
#endif

template <bool kHandoff, bool kPeer>
__global__ void __maxnreg__(kMaxRegisters)
decode_splitkv_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                      const DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);  // [kGroups][kStages]
    uint64_t* empty = full + kGroups * kStages;
    int* flag = reinterpret_cast<int*>(empty + kStages);
    uint8_t* staging = kHandoff ? smem : smem + kStages * kStageBytes + kBarrierBytes;
    float* stage_o = reinterpret_cast<float*>(staging + (kHandoff ? AB_DECODE_O_OFFSET_BYTES : 0));
    float* stage_lse = reinterpret_cast<float*>(staging + (kHandoff ? AB_DECODE_LSE_OFFSET_BYTES : 2048));

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_heads = p.kv_heads * kGroup;
#ifdef TC_TRACE
    __shared__ unsigned int trace_cta;
    const unsigned long long trace_entry = tc::global_timer_ns();
    if (threadIdx.x == 0) trace_cta = atomicAdd(&g_trace_ctas, 1u);
#endif

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            for (int g = 0; g < kGroups; ++g) tc::mbar_init(&full[g * kStages + s], 1);
            tc::mbar_init(&empty[s], kGroupWarps);
        }
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&kmap);
        tc::tma_prefetch_desc(&vmap);
    }
    // Programmatic dependent launch: everything above touches only this CTA's shared memory and
    // kernel parameters, so it may overlap the tail of the preceding kernel in the stream. Nothing
    // below (lengths, caches, tickets) is read before that kernel has completed. The next kernel
    // may start its own preamble as soon as every CTA of this grid is resident.
    // With cache_stable the lengths, the index tables and the K/V rows may be read at once; q, the new
    // rows and every write still wait (further down, consumer warps only).
    if (!p.cache_stable) {
        tc::grid_dependency_wait();
        tc::grid_launch_dependents();
    }

    // Device-side lengths: no host read. Values outside the contract are clamped so that no
    // address leaves the cache.
    int64_t old_len = p.old_lengths[b];
    old_len = old_len < 0 ? 0 : old_len;
    const int64_t visible_global = old_len + (p.append ? 1 : 0);
    int64_t visible_local = visible_global - p.shard_start;
    visible_local = visible_local < 0 ? 0 : (visible_local > p.capacity ? p.capacity : visible_local);
    const int n_valid = int(visible_local);
    const int64_t append_local = old_len - p.shard_start;
    const bool do_append = p.append && append_local >= 0 && append_local < p.capacity;
    const int append_row = do_append ? int(append_local) : -1;
    int slot_of_b = b;
    if (p.cache_batch_idx) {
        slot_of_b = __ldg(p.cache_batch_idx + b);
        slot_of_b = slot_of_b < 0 ? 0 : (slot_of_b >= p.cache_slots ? p.cache_slots - 1 : slot_of_b);
    }

    const int tiles = (n_valid + kTileN - 1) / kTileN;
    const int tile_begin = int((int64_t(split) * tiles) / p.splits);
    const int tile_end = int((int64_t(split + 1) * tiles) / p.splits);
    const int n_tiles = tile_end - tile_begin;

    __syncthreads();
#ifdef TC_TRACE
    unsigned long long* trace_row = (threadIdx.x == 0 || (warp == kConsumerWarps && lane == 0)) ? g_trace[trace_cta % 1024u] : nullptr;
    if (threadIdx.x == 0) {
        unsigned int sm;
        asm("mov.u32 %0, %%smid;" : "=r"(sm));
        trace_row[0] = trace_entry;
        trace_row[1] = trace_cta;
        trace_row[2] = (unsigned long long)(split | (kvh << 8) | (n_tiles << 16));
        trace_row[23] = sm;
        trace_row[3] = tc::global_timer_ns();
    }
#endif
    if (p.cache_stable && (warp != kConsumerWarps || (p.cache_stable == 2 && p.block_table))) {
        // (a paged cache under the narrower promise streams nothing early: its producer waits as well)
        tc::grid_dependency_wait();
        tc::grid_launch_dependents();  // after the wait: the next launch can overlap this one only
        TC_TRACE_POINT(27);
    }

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer warp
        const uint64_t policy = tc::policy_evict_first();
        // Tiles [0, early_tiles) of this CTA hold only rows the caller promised stable: they may be fetched
        // before the stream dependency resolves. The ring takes the first kStages of them; the rest are
        // prefetched into L2, from where they arrive at L2 speed once the consumers free ring stages.
        int early_tiles = 0;
        if (p.cache_stable == 1) {
            early_tiles = n_tiles;
        } else if (p.cache_stable == 2) {
            const int64_t touched = old_len - 1 - p.shard_start;  // the one row the preceding kernel may have written
            const int64_t stable_end = touched < 0 ? 0 : touched / kTileN;
            const int64_t count = stable_end - tile_begin;
            early_tiles = int(count < 0 ? 0 : (count > n_tiles ? n_tiles : count));
        }
        // A long share gains nothing from an early start (its launch is bandwidth-bound from end to end) and the
        // early reads compete with the preceding launch's stream: config 5 ran 5 % slower with them.
        if (n_tiles > kEarlyLimitTiles) early_tiles = 0;
        auto issue_tile = [&](int it, int slot, int row0) {
            const int stage = (n_tiles - 1 - it) % kStages;  // the last tile always lands in stage 0
            const uint32_t generation = uint32_t(it / kStages);
            if (!tc::mbar_wait(&empty[stage], (generation & 1) ^ 1)) {
                atomicCAS(p.status, 0, 1);
                return false;
            }
            uint8_t* base = smem + stage * kStageBytes;
            uint64_t* landed = &full[((n_tiles - 1 - it) % kGroups) * kStages + stage];  // the owning group's barrier
            tc::mbar_arrive_expect_tx(landed, kStageBytes);
            tc::tma_load_4d(base, &vmap, landed, 0, kvh, row0, slot, policy);
            tc::tma_load_4d(base + kHalfBytes, &vmap, landed, 64, kvh, row0, slot, policy);
            tc::tma_load_4d(base + kVBytes, &kmap, landed, 0, kvh, row0, slot, policy);
            tc::tma_load_4d(base + kVBytes + kHalfBytes, &kmap, landed, 64, kvh, row0, slot, policy);
            return true;
        };
        if (!p.block_table) {
            if (lane == 0) {
                const int ring_early = early_tiles < kStages ? early_tiles : kStages;
                bool ok = true;
                int it = 0;
                for (; ok && it < ring_early; ++it) ok = issue_tile(it, slot_of_b, (tile_begin + it) * kTileN);
                TC_TRACE_POINT(24);
                // Only a share of at most kPrefetchTiles beyond the ring is prefetched (about 55 MB over a full
                // grid, so it is still in the 126 MB L2 when its turn comes). A longer share streams at the HBM
                // rate anyway, and prefetching a part of it only disturbed that stream when measured.
                const int prefetch_end = early_tiles <= kStages + kPrefetchTiles ? early_tiles : kStages;
                for (int ahead = kStages; ahead < prefetch_end; ++ahead) {
                    const int row0 = (tile_begin + ahead) * kTileN;
                    tc::tma_prefetch_4d(&vmap, 0, kvh, row0, slot_of_b);
                    tc::tma_prefetch_4d(&vmap, 64, kvh, row0, slot_of_b);
                    tc::tma_prefetch_4d(&kmap, 0, kvh, row0, slot_of_b);
                    tc::tma_prefetch_4d(&kmap, 64, kvh, row0, slot_of_b);
                }
                TC_TRACE_POINT(25);
                for (; ok && it < n_tiles; ++it) {
                    // A tile outside the promise is fetched only after the preceding kernel has completed.
                    if (p.cache_stable && it == early_tiles) tc::grid_dependency_wait();
                    ok = issue_tile(it, slot_of_b, (tile_begin + it) * kTileN);
                }
                TC_TRACE_POINT(26);
            }
        } else {
            // Paged cache: the whole warp looks up the pages of the next 32 tiles with one coalesced
            // load, so the table's latency is paid once per 32 tiles and not once per tile.
            if (p.cache_stable == 1 && early_tiles == 0) tc::grid_dependency_wait();  // a long share starts late
            bool ok = true;
            for (int first = 0; first < n_tiles && ok; first += 32) {
                int slot = 0, local = 0;
                if (first + lane < n_tiles) locate_row(p, b, slot_of_b, (tile_begin + first + lane) * kTileN, slot, local);
                const int count = min(32, n_tiles - first);
                for (int j = 0; j < count && ok; ++j) {
                    const int tile_slot = __shfl_sync(0xffffffffu, slot, j);
                    const int tile_row0 = __shfl_sync(0xffffffffu, local, j);
                    if (lane == 0) ok = issue_tile(first + j, tile_slot, tile_row0);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                }
            }
        }
        if (p.cache_stable) tc::grid_launch_dependents();
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const int qrow = lane >> 2;       // query head within the group; rows >= 4 are padding
    const int quad = lane & 3;
    const bool row_ok = qrow < kGroup;
    uint32_t qa[8][2];
    {
        const uint32_t* qptr = reinterpret_cast<const uint32_t*>(
            p.q + (int64_t(b) * q_heads + kvh * kGroup + (row_ok ? qrow : 0)) * kDim);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qa[ks][0] = row_ok ? __ldg(qptr + ks * 8 + quad) : 0u;
            qa[ks][1] = row_ok ? __ldg(qptr + ks * 8 + 4 + quad) : 0u;
        }
        if (p.rope_cos && row_ok) {
            // This thread holds columns 16*ks + 2*quad + {0,1} and + 8 + {0,1}; the partner of column
            // i < 64 is i + 64, i.e. the same slot of fragment ks + 4: the rotation is thread-local.
            int64_t position = old_len < p.rope_positions ? old_len : p.rope_positions - 1;
            const float2* cos2 = reinterpret_cast<const float2*>(p.rope_cos + position * 64);
            const float2* sin2 = reinterpret_cast<const float2*>(p.rope_sin + position * 64);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int pair = ks * 8 + half * 4 + quad;  // columns 2*pair, 2*pair + 1
                    const float2 c = __ldg(cos2 + pair), sn = __ldg(sin2 + pair);
                    const uint32_t lo = qa[ks][half], hi = qa[ks + 4][half];
                    float lo0, hi0, lo1, hi1;
                    rope_pair(bf16_lo(lo), bf16_lo(hi), c.x, sn.x, lo0, hi0);
                    rope_pair(bf16_hi(lo), bf16_hi(hi), c.y, sn.y, lo1, hi1);
                    qa[ks][half] = tc::pack_bf16x2(lo0, lo1);
                    qa[ks + 4][half] = tc::pack_bf16x2(hi0, hi1);
                }
            }
        }
    }
    // Accumulators of query rows 0-7 only (rows 4-7 are padding, rows 8-15 of the MMA tile are fed zeros).
    float o[16][2];
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = 0.f;
    float row_max = -INFINITY, row_sum = 0.f;
    bool failed = false;
    // Tile `it` belongs to group (n_tiles - 1 - it) % kGroups: the last tile, which lands in stage 0, to group 0,
    // the one before it (stage 1) to group 1. A group's last tile therefore sits in the stage of its own number.
    const int group = warp / kGroupWarps, gw = warp % kGroupWarps;
    const int first_tile = (((n_tiles - 1 - group) % kGroups) + kGroups) % kGroups;

    for (int it = first_tile; it < n_tiles; it += kGroups) {
        const int stage = (n_tiles - 1 - it) % kStages;
        if (!tc::mbar_wait(&full[group * kStages + stage], uint32_t(it / kRingPeriod) & 1)) {
            failed = true;
            break;
        }
        if (it < 8) TC_TRACE_POINT(4 + 2 * it);
        uint8_t* vbase = smem + stage * kStageBytes;
        uint8_t* kbase = vbase + kVBytes;
        const int tile_row0 = (tile_begin + it) * kTileN;
        const int warp_row0 = tile_row0 + gw * 16;  // first cache row owned by this warp
        const int valid = n_valid - warp_row0;         // >= 16: all of this warp's keys are visible

        if (append_row >= warp_row0 && append_row < warp_row0 + 16) {
            // Fused append: the new row goes to both caches and patches this tile in shared memory,
            // so the value the TMA copy fetched for that row never matters.
            const uint32_t r = uint32_t(append_row - tile_row0);
            const int chunk = lane & 15;
            const bool is_v = lane >= 16;
            uint4 value = __ldg(reinterpret_cast<const uint4*>(
                (is_v ? p.vnew : p.knew) + (int64_t(b) * p.kv_heads + kvh) * kDim) + chunk);
            if (p.rope_cos) {
                // Lanes 0-7 hold K columns [8*lane, 8*lane + 8), lanes 8-15 their partners 64 further on.
                uint4 other;
                other.x = __shfl_xor_sync(0xffffffffu, value.x, 8);
                other.y = __shfl_xor_sync(0xffffffffu, value.y, 8);
                other.z = __shfl_xor_sync(0xffffffffu, value.z, 8);
                other.w = __shfl_xor_sync(0xffffffffu, value.w, 8);
                if (!is_v) {
                    const bool upper = chunk >= 8;
                    int64_t position = old_len < p.rope_positions ? old_len : p.rope_positions - 1;
                    const float4* cos4 = reinterpret_cast<const float4*>(p.rope_cos + position * 64) + (chunk & 7) * 2;
                    const float4* sin4 = reinterpret_cast<const float4*>(p.rope_sin + position * 64) + (chunk & 7) * 2;
                    const float4 c0 = __ldg(cos4), c1 = __ldg(cos4 + 1), s0 = __ldg(sin4), s1 = __ldg(sin4 + 1);
                    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                    const uint32_t mine[4] = {value.x, value.y, value.z, value.w};
                    const uint32_t theirs[4] = {other.x, other.y, other.z, other.w};
                    uint32_t rotated[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t lo = upper ? theirs[j] : mine[j], hi = upper ? mine[j] : theirs[j];
                        float lo0, hi0, lo1, hi1;
                        rope_pair(bf16_lo(lo), bf16_lo(hi), c[2 * j], sn[2 * j], lo0, hi0);
                        rope_pair(bf16_hi(lo), bf16_hi(hi), c[2 * j + 1], sn[2 * j + 1], lo1, hi1);
                        rotated[j] = upper ? tc::pack_bf16x2(hi0, hi1) : tc::pack_bf16x2(lo0, lo1);
                    }
                    value = make_uint4(rotated[0], rotated[1], rotated[2], rotated[3]);
                }
            }
            *reinterpret_cast<uint4*>((is_v ? vbase : kbase) + swizzled(r, chunk)) = value;
            __nv_bfloat16* cache = is_v ? p.vcache : p.kcache;
            int slot, local;
            locate_row(p, b, slot_of_b, append_row, slot, local);
            reinterpret_cast<uint4*>(cache + ((int64_t(slot) * p.page_size + local) * p.kv_heads + kvh) * kDim)[chunk] =
                value;
            tc::fence_proxy_async_smem();
            __syncwarp();
        }
        if (valid < 16) {
            // Rows past the visible length may hold anything (NaN included): zero V so that
            // 0 * garbage cannot reach the accumulator. K garbage is masked by index below.
            const int first = valid < 0 ? 0 : valid;
            for (int idx = lane; idx < 256; idx += 32) {
                const int rr = idx >> 4;
                if (rr >= first)
                    *reinterpret_cast<uint4*>(vbase + swizzled(uint32_t(gw * 16 + rr), uint32_t(idx & 15))) =
                        make_uint4(0, 0, 0, 0);
            }
            tc::fence_proxy_async_smem();
            __syncwarp();
        }

        if (valid > 0) {
            float s[2][2];
#pragma unroll
            for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = 0.f;
            const uint32_t kaddr = tc::smem_u32(kbase);
            const uint32_t vaddr = tc::smem_u32(vbase);
            const int mat = lane >> 3, mrow = lane & 7;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                // matrices: (keys 0-7, d lo) (keys 0-7, d hi) (keys 8-15, d lo) (keys 8-15, d hi)
                const uint32_t r = uint32_t(gw * 16 + (mat >> 1) * 8 + mrow);
                const uint32_t chunk = uint32_t(ks * 2 + (mat & 1));
                uint32_t b00, b01, b10, b11;
                tc::ldmatrix_x4(kaddr + swizzled(r, chunk), b00, b01, b10, b11);
                tc::mma_bf16_16816_rows8(s[0][0], s[0][1], qa[ks][0], qa[ks][1], b00, b01);
                tc::mma_bf16_16816_rows8(s[1][0], s[1][1], qa[ks][0], qa[ks][1], b10, b11);
            }
            if (valid < 16) {
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int e = 0; e < 2; ++e)
                        if (n * 8 + quad * 2 + e >= valid) s[n][e] = -INFINITY;
            }
            float tile_max = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
            tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
            tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
            const float new_max = fmaxf(row_max, tile_max);  // finite: key 0 of this warp is visible
            const float alpha = tc::fast_exp2((row_max - new_max) * p.scale_log2);
            const float bias = new_max * p.scale_log2;
            float pr[2][2];
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) pr[n][e] = tc::fast_exp2(fmaf(s[n][e], p.scale_log2, -bias));
            row_sum = fmaf(row_sum, alpha, (pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]));
            row_max = new_max;
#pragma unroll
            for (int n = 0; n < 16; ++n) {
                o[n][0] *= alpha;
                o[n][1] *= alpha;
            }
            const uint32_t pa0 = row_ok ? tc::pack_bf16x2(pr[0][0], pr[0][1]) : 0u;
            const uint32_t pa2 = row_ok ? tc::pack_bf16x2(pr[1][0], pr[1][1]) : 0u;
#pragma unroll
            for (int np = 0; np < 8; ++np) {
                // matrices: (keys 0-7, d n0) (keys 8-15, d n0) (keys 0-7, d n0+1) (keys 8-15, d n0+1)
                const uint32_t r = uint32_t(gw * 16 + (mat & 1) * 8 + mrow);
                const uint32_t chunk = uint32_t(np * 2 + (mat >> 1));
                uint32_t v00, v01, v10, v11;
                tc::ldmatrix_x4_trans(vaddr + swizzled(r, chunk), v00, v01, v10, v11);
                tc::mma_bf16_16816_rows8(o[2 * np][0], o[2 * np][1], pa0, pa2, v00, v01);
                tc::mma_bf16_16816_rows8(o[2 * np + 1][0], o[2 * np + 1][1], pa0, pa2, v10, v11);
            }
        }
        __syncwarp();
        if (it < 8) TC_TRACE_POINT(5 + 2 * it);
        if (it + 1 < n_tiles && lane == 0) tc::mbar_arrive(&empty[stage]);
    }
    if (failed) atomicCAS(p.status, 0, 2);
    TC_TRACE_POINT(20);

    // ---------------------------------------------------------------------- CTA epilogue
    // Quad-partial row sums become full sums; each warp parks its partial in the K rows it owns in its
    // group's terminal stage (nobody else reads those rows: the group is done with them and the other
    // group never reads that stage again), then one barrier releases the stages.
    row_sum += __shfl_xor_sync(0xffffffffu, row_sum, 1);
    row_sum += __shfl_xor_sync(0xffffffffu, row_sum, 2);
    uint8_t* terminal_k = smem + kVBytes;  // K tile of stage 0; group g parks in the K tile of stage g
    uint8_t* group_k = terminal_k + group * kStageBytes;
    float* part_o = reinterpret_cast<float*>(group_k + gw * 2048);                 // [4][128]
    float* part_ml = reinterpret_cast<float*>(group_k + kHalfBytes + gw * 2048);   // [4][2]
    if (row_ok) {
#pragma unroll
        for (int n = 0; n < 16; ++n)
            *reinterpret_cast<float2*>(part_o + qrow * kDim + n * 8 + quad * 2) = make_float2(o[n][0], o[n][1]);
        if (quad == 0) *reinterpret_cast<float2*>(part_ml + qrow * 2) = make_float2(row_max, row_sum);
    }
    consumer_barrier();  // all K/V readers are done: the terminal V region changes owner here
    if (threadIdx.x >= kMergeThreads) return;  // the epilogue is the work of four warps

    const int tid = threadIdx.x;
    const int row = tid >> 5;        // query head within the group
    const int col4 = tid & 31;       // float4 column
    {
        float m_w[kConsumerWarps], l_w[kConsumerWarps];
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
            const uint8_t* parked = terminal_k + (w / kGroupWarps) * kStageBytes + (w % kGroupWarps) * 2048;
            const float2 ml = *reinterpret_cast<const float2*>(parked + kHalfBytes + row * 8);
            m_w[w] = ml.x;
            l_w[w] = ml.y;
            m_all = fmaxf(m_all, ml.x);
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float l_all = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
            const float weight = m_w[w] == -INFINITY ? 0.f : tc::fast_exp2((m_w[w] - m_all) * p.scale_log2);
            const float4 v = *reinterpret_cast<const float4*>(
                terminal_k + (w / kGroupWarps) * kStageBytes + (w % kGroupWarps) * 2048 + row * 512 + col4 * 16);
            l_all = fmaf(weight, l_w[w], l_all);
            acc.x = fmaf(weight, v.x, acc.x);
            acc.y = fmaf(weight, v.y, acc.y);
            acc.z = fmaf(weight, v.z, acc.z);
            acc.w = fmaf(weight, v.w, acc.w);
        }
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
        *reinterpret_cast<float4*>(stage_o + row * kDim + col4 * 4) = acc;
        if (col4 == 0) stage_lse[row] = l_all > 0.f ? fmaf(m_all, p.scale, logf(l_all)) : -INFINITY;
    }
    merge_barrier();  // publish the four output rows and their LSE together
    TC_TRACE_POINT(21);

    const int64_t head_slot = int64_t(b) * p.kv_heads + kvh;  // index of the (batch, KV head) pair
    float4 final_o;
    float final_lse;
    if (p.splits > 1) {
        // Vector export of the staged tile: one 16-byte word per thread.
        const int64_t slot = int64_t(split) * p.batch * p.kv_heads + head_slot;
        reinterpret_cast<uint4*>(p.ws_o + slot * (kGroup * kDim))[tid] = reinterpret_cast<const uint4*>(stage_o)[tid];
        if (tid == 0)
            *reinterpret_cast<uint4*>(p.ws_lse + slot * kGroup) = *reinterpret_cast<const uint4*>(stage_lse);
        // The barrier orders every thread's partial stores before thread 0's release; the last
        // arriver's acquire, followed by the second barrier, orders them before the merge loads.
        merge_barrier();
        if (tid == 0) *flag = tc::atomic_add_acq_rel(p.tickets + head_slot, 1) == p.splits - 1;
        merge_barrier();
        TC_TRACE_POINT(22);
        if (!*flag) return;
        // Last CTA of this (batch, KV head): LSE-weighted merge of every split's partial. Warp w owns
        // output row w: its lanes first fetch that row's split LSEs together (one L2 round trip),
        // reduce them with shuffles and park the weights in the released terminal K stage; then
        // each lane accumulates its four columns over the splits, with the first batch of partial-O
        // loads already in flight beside the LSE loads.
        const int64_t stride_lse = int64_t(p.batch) * p.kv_heads * kGroup;
        const float* lse_base = p.ws_lse + head_slot * kGroup + row;
        const float4* o_base = reinterpret_cast<const float4*>(p.ws_o + head_slot * (kGroup * kDim) + row * kDim) + col4;
        const int64_t stride_o4 = stride_lse * (kDim / 4);
        float* weights = reinterpret_cast<float*>(terminal_k) + row * kMaxSplits;
        constexpr int kBatch = 20;  // partial-O loads kept in flight per lane
        float part_lse[kMaxSplits / 32];
        float4 v[kBatch];
#pragma unroll
        for (int i = 0; i < kMaxSplits / 32; ++i) {
            const int s = col4 + 32 * i;
            part_lse[i] = s < p.splits ? __ldcg(lse_base + s * stride_lse) : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u)  // first batch goes out with the LSE loads: one L2 round trip
            if (u < p.splits) v[u] = __ldcg(o_base + u * stride_o4);
        float lse_max = -INFINITY;
#pragma unroll
        for (int i = 0; i < kMaxSplits / 32; ++i) lse_max = fmaxf(lse_max, part_lse[i]);
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1)
            lse_max = fmaxf(lse_max, __shfl_xor_sync(0xffffffffu, lse_max, offset));
        TC_TRACE_POINT(28);
        float total = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxSplits / 32; ++i) {
            const float weight = part_lse[i] == -INFINITY ? 0.f : __expf(part_lse[i] - lse_max);
            weights[col4 + 32 * i] = weight;
            total += weight;
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) total += __shfl_xor_sync(0xffffffffu, total, offset);
        __syncwarp();
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < p.splits; s0 += kBatch) {
            if (s0 > 0) {
#pragma unroll
                for (int u = 0; u < kBatch; ++u)
                    if (s0 + u < p.splits) v[u] = __ldcg(o_base + (s0 + u) * stride_o4);
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const float w = s0 + u < p.splits ? weights[s0 + u] : 0.f;
                if (w > 0.f) {  // a split that saw no key may hold anything: never multiply it
                    acc.x = fmaf(w, v[u].x, acc.x);
                    acc.y = fmaf(w, v[u].y, acc.y);
                    acc.z = fmaf(w, v[u].z, acc.z);
                    acc.w = fmaf(w, v[u].w, acc.w);
                }
            }
        }
        TC_TRACE_POINT(29);
        const float inv = total > 0.f ? 1.f / total : 0.f;
        final_o = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        final_lse = total > 0.f ? lse_max + logf(total) : -INFINITY;
        // Every split of this head has taken its ticket: a plain store re-arms the counter for the next launch
        // (an atomic exchange would keep this CTA, and with it the end of the kernel, waiting for its return).
        if (tid == 0) p.tickets[head_slot] = 0;
    } else {
        final_o = *reinterpret_cast<const float4*>(stage_o + row * kDim + col4 * 4);
        final_lse = stage_lse[row];
    }

    const int64_t out_row = int64_t(b) * q_heads + kvh * kGroup + row;
    if (kPeer) {
        // Cross-GPU merge inside the same launch. This CTA holds this rank's partial for the
        // (batch, KV head) unit. Every thread stores its 16 bytes of the partial, each 4-byte value
        // paired with the call's epoch, into every rank's exchange block (plain peer stores over
        // NVLink, its own block included), then polls its own block until the words of every source
        // rank carry this epoch (bounded), and merges. No fence, barrier or separate flag sits between
        // the store and the remote read. Slots alternate with the epoch's parity: a rank can be at
        // most one call ahead of the slowest reader, because it cannot finish call e+1 before that
        // reader has stored its own e+1 partial, which it does only after it has merged call e.
        const int world = p.world, units = p.batch * p.kv_heads, unit = int(head_slot);
        uint8_t* mine = p.peer_blocks[p.rank];
        uint32_t* epochs = reinterpret_cast<uint32_t*>(mine + peer_epochs_offset(world, units));
        const uint32_t epoch = epochs[unit] + 1;  // only this CTA touches the word during this launch
        const size_t slot_bytes = (size_t(epoch & 1) * world * units + unit) * kPeerSlotBytes;
        const size_t rank_stride = size_t(units) * kPeerSlotBytes;
        for (int r = 0; r < world; ++r) {
            uint8_t* slot = p.peer_blocks[r] + slot_bytes + p.rank * rank_stride;
            tc::store_flagged_2(slot + tid * 32, __float_as_uint(final_o.x), __float_as_uint(final_o.y), epoch);
            tc::store_flagged_2(slot + tid * 32 + 16, __float_as_uint(final_o.z), __float_as_uint(final_o.w), epoch);
            if (col4 == 0) tc::store_flagged_1(slot + kPeerLseOffset + row * 8, __float_as_uint(final_lse), epoch);
        }
        float4 part_o[kMaxPeers];
        float part_lse[kMaxPeers];
#pragma unroll
        for (int s = 0; s < kMaxPeers; ++s) {
            part_o[s] = make_float4(0.f, 0.f, 0.f, 0.f);
            part_lse[s] = -INFINITY;
        }
        uint32_t pending = (1u << world) - 1u;
        const uint8_t* arrivals = mine + slot_bytes;
        const uint64_t wait_start = tc::global_timer_ns();
        for (uint32_t poll = 1; pending; ++poll) {
#pragma unroll
            for (int s = 0; s < kMaxPeers; ++s) {
                if ((pending >> s) & 1u) {
                    const uint8_t* slot = arrivals + s * rank_stride;
                    const uint4 lo = tc::load_volatile_16(slot + tid * 32), hi = tc::load_volatile_16(slot + tid * 32 + 16);
                    const uint2 l = tc::load_volatile_8(slot + kPeerLseOffset + row * 8);
                    if (lo.y == epoch && lo.w == epoch && hi.y == epoch && hi.w == epoch && l.y == epoch) {
                        part_o[s] = make_float4(__uint_as_float(lo.x), __uint_as_float(lo.z), __uint_as_float(hi.x),
                                                __uint_as_float(hi.z));
                        part_lse[s] = __uint_as_float(l.x);
                        pending &= ~(1u << s);
                    }
                }
            }
            if (pending && (poll & 15u) == 0 && tc::global_timer_ns() - wait_start > TC_WAIT_LIMIT_NS) {
                atomicCAS(p.status, 0, 5);  // a rank never delivered: the result below is not valid
                break;
            }
        }
        float4 merged;
        float merged_lse;
        lse_weighted_merge<kMaxPeers>(
            world, [&](int s) { return part_lse[s]; }, [&](int s) { return part_o[s]; }, merged, merged_lse);
        uint2 packed;
        packed.x = tc::pack_bf16x2(merged.x, merged.y);
        packed.y = tc::pack_bf16x2(merged.z, merged.w);
        *reinterpret_cast<uint2*>(p.out + out_row * kDim + col4 * 4) = packed;
        if (col4 == 0) p.lse[out_row] = merged_lse;
        merge_barrier();  // every thread has read the unit's epoch before it moves on
        if (tid == 0) epochs[unit] = epoch;
    } else if (p.partial) {
        *reinterpret_cast<float4*>(p.partial_o + out_row * kDim + col4 * 4) = final_o;
        if (col4 == 0) p.lse[out_row] = final_lse;
    } else {
        uint2 packed;
        packed.x = tc::pack_bf16x2(final_o.x, final_o.y);
        packed.y = tc::pack_bf16x2(final_o.z, final_o.w);
        *reinterpret_cast<uint2*>(p.out + out_row * kDim + col4 * 4) = packed;
        if (col4 == 0) p.lse[out_row] = final_lse == -INFINITY ? INFINITY : final_lse;
    }
    TC_TRACE_POINT(19);
}

// Standalone merge of `parts` partial results (used after the multi-GPU all-gather).
__global__ void __launch_bounds__(128) combine_partials_kernel(const float* __restrict__ partial_o,
                                                               const float* __restrict__ partial_lse, int parts,
                                                               int64_t rows, int64_t stride_o, int64_t stride_lse,
                                                               __nv_bfloat16* __restrict__ out,
                                                               float* __restrict__ lse) {
    const int64_t row = int64_t(blockIdx.x) * 4 + (threadIdx.x >> 5);
    const int col4 = threadIdx.x & 31;
    if (row >= rows) return;
    float4 merged;
    float merged_lse;
    lse_weighted_merge<0>(
        parts, [&](int s) { return partial_lse[s * stride_lse + row]; },
        [&](int s) { return reinterpret_cast<const float4*>(partial_o + s * stride_o + row * kDim)[col4]; }, merged,
        merged_lse);
    uint2 packed;
    packed.x = tc::pack_bf16x2(merged.x, merged.y);
    packed.y = tc::pack_bf16x2(merged.z, merged.w);
    *reinterpret_cast<uint2*>(out + row * kDim + col4 * 4) = packed;
    if (col4 == 0) lse[row] = merged_lse;
}

// ------------------------------------------------------------------------------- host side
int auto_splits(const tc::DeviceInfo& info, int64_t batch, int64_t capacity, int64_t kv_heads) {
    // About one CTA per SM (the second resident CTA slot is left to the next launch's preamble and to
    // uneven split lengths); the merge tail grows with the split count, so more is not better.
    const int64_t slots = int64_t(info.sms);
    int64_t splits = slots / (batch * kv_heads);
    const int64_t tiles = (capacity + kTileN - 1) / kTileN;
    if (splits > tiles) splits = tiles;
    if (splits > kMaxSplits) splits = kMaxSplits;
    if (splits < 1) splits = 1;
    return int(splits);
}

int check_geometry(int device, int64_t batch, int64_t capacity, int64_t kv_heads, int64_t num_splits,
                   int64_t mapping, int append, tc::DeviceInfo* info, int* splits) {
    int status = tc::require_sm100(device, info);
    if (status != TC_OK) return status;
    TC_REQUIRE(mapping == 0 || mapping == 1, "Expected mapping 0 (dedicated staging) or 1 (planner handoff)");
    TC_REQUIRE(batch > 0 && batch <= 65535, "Q must be [B,1,Hq,128] with 1 <= B <= 65535");
    TC_REQUIRE(kv_heads >= 1 && kv_heads <= 8, "caches must be [B,C,Hkv,128] with 1 <= Hkv <= 8");
    TC_REQUIRE(capacity >= 4, "Full capacity cache must be [B,C>=4,Hkv,128]");
    TC_REQUIRE(capacity <= (int64_t(1) << 30), "cache capacity overflows the kernel's int geometry");
    TC_REQUIRE(batch * kv_heads <= tc::kTicketSlots, "B*Hkv exceeds the library's ticket block");
    TC_REQUIRE(num_splits >= 0 && num_splits <= kMaxSplits, "num_splits must be 0 (auto) or in [1,128]");
    (void)append;
    *splits = num_splits > 0 ? int(num_splits) : auto_splits(*info, batch, capacity, kv_heads);
    return TC_OK;
}

template <bool kHandoff, bool kPeer = false>
int launch(const CUtensorMap& kmap, const CUtensorMap& vmap, const DecodeParams& p, cudaStream_t stream) {
    auto kernel = &decode_splitkv_kernel<kHandoff, kPeer>;
    constexpr int shared = shared_bytes(kHandoff);
    static thread_local int configured_device = -1;
    int device = 0;
    TC_CUDA(cudaGetDevice(&device));
    if (configured_device != device) {
        TC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared));
        configured_device = device;
    }
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(p.splits, p.kv_heads, p.batch);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    TC_CUDA(cudaLaunchKernelEx(&config, kernel, kmap, vmap, p));
    return TC_OK;
}

struct PeerArgs {
    void* const* blocks;  // world pointers: every rank's exchange block as mapped into this process
    int world, rank;
};

struct RopeTables {
    const float* cos;  // fp32 [positions, 64]
    const float* sin;
    int64_t positions;
};

struct IndexedCache {
    const int32_t* block_table;     // [B, pages_per_seq] (row stride table_stride) or nullptr
    int64_t table_stride, pages_per_seq;
    const int32_t* cache_batch_idx;  // [B] or nullptr
    int64_t cache_slots;             // pages, or batch entries of the cache tensors
    int64_t slot_rows;               // rows per slot: the page size, or the capacity
};

struct MapKey {
    const void* base;
    int64_t batch, capacity, kv_heads;
    int device;
    bool operator==(const MapKey& other) const {
        return base == other.base && batch == other.batch && capacity == other.capacity &&
               kv_heads == other.kv_heads && device == other.device;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& key) const {
        return std::hash<const void*>()(key.base) ^ (std::hash<int64_t>()(key.capacity) * 31) ^
               (std::hash<int64_t>()(key.batch * 16 + key.kv_heads) * 131) ^ size_t(key.device);
    }
};

// Encoding a tensor map costs a few microseconds of host time, comparable to the kernel itself at
// short lengths, so maps are memoised per (pointer, geometry).
int cache_map(int device, const void* base, int64_t batch, int64_t capacity, int64_t kv_heads, CUtensorMap* out) {
    static std::mutex lock;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{base, batch, capacity, kv_heads, device};
    std::lock_guard<std::mutex> guard(lock);
    auto found = cache.find(key);
    if (found == cache.end()) {
        if (cache.size() > 4096) cache.clear();
        CUtensorMap map;
        int status = tc::make_rows_map(&map, base, false, kv_heads, capacity, batch, kDim, kv_heads * kDim,
                                       capacity * kv_heads * kDim, kTileN, 2);
        if (status != TC_OK) return status;
        found = cache.emplace(key, map).first;
    }
    *out = found->second;
    return TC_OK;
}

int decode_common(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                  const void* vnew, const int32_t* old_lengths, void* out, float* lse, float* partial_o,
                  float* workspace_o, int64_t workspace_o_elems, float* workspace_lse, int64_t workspace_lse_elems,
                  int64_t batch, int64_t capacity, int64_t kv_heads, int64_t num_splits, int64_t mapping, int append,
                  int partial, int64_t shard_start, const PeerArgs* peer = nullptr,
                  const IndexedCache* indexed = nullptr, const RopeTables* rope = nullptr, int cache_stable = 0) {
    tc::DeviceInfo info;
    int splits = 1;
    int status = check_geometry(device, batch, capacity, kv_heads, num_splits, mapping, append, &info, &splits);
    if (status != TC_OK) return status;
    TC_REQUIRE(q && kcache && vcache && knew && vnew && old_lengths && lse && (partial == 1 ? (void*)partial_o : out),
               "null tensor pointer");
    TC_REQUIRE(shard_start >= 0, "kv_shard_start must be non-negative");
    TC_REQUIRE((partial == 2) == (peer != nullptr), "peer exchange arguments do not match the call");
    if (peer) {
        TC_REQUIRE(peer->world >= 1 && peer->world <= kMaxPeers && peer->rank >= 0 && peer->rank < peer->world,
                   "peer exchange needs 1 <= world <= 8 and 0 <= rank < world");
        TC_REQUIRE(peer->blocks, "null peer block table");
        for (int r = 0; r < peer->world; ++r)
            TC_REQUIRE(peer->blocks[r] && reinterpret_cast<uintptr_t>(peer->blocks[r]) % 16 == 0,
                       "every rank's exchange block must be mapped and 16-byte aligned");
        // Every CTA of the grid must be resident at once: a CTA that waits for another rank holds
        // its slot, and the CTAs it indirectly waits for on that rank must never queue behind waiters.
        TC_REQUIRE(int64_t(splits) * kv_heads * batch <= int64_t(info.sms) * AB_DECODE_CTAS_PER_SM,
                   "peer exchange needs splits*Hkv*B CTAs to be co-resident; lower num_splits");
    }
    const int64_t q_heads = kv_heads * kGroup;
    const int64_t rows = batch * q_heads;
    const int64_t cache_slots = indexed ? indexed->cache_slots : batch;
    const int64_t slot_rows = indexed ? indexed->slot_rows : capacity;
    if (indexed) {
        TC_REQUIRE(!(indexed->block_table && indexed->cache_batch_idx),
                   "a paged cache is indexed by its block table only: cache_batch_idx must be null");
        TC_REQUIRE(partial == 0 && shard_start == 0, "indexed caches are not combined with KV-sequence sharding");
        TC_REQUIRE(cache_slots >= 1 && cache_slots <= (int64_t(1) << 30) && slot_rows >= 4, "cache tensor geometry out of range");
        if (indexed->block_table) {
            TC_REQUIRE(slot_rows % kTileN == 0, "page size must be a multiple of 64 rows");
            TC_REQUIRE(indexed->pages_per_seq >= 1 && indexed->table_stride >= indexed->pages_per_seq &&
                           capacity == indexed->pages_per_seq * slot_rows,
                       "block table must be [B, pages_per_seq] with capacity = pages_per_seq * page_size");
            TC_REQUIRE(reinterpret_cast<uintptr_t>(indexed->block_table) % 4 == 0, "misaligned block table");
        } else {
            TC_REQUIRE(indexed->cache_batch_idx && slot_rows == capacity, "cache_batch_idx required");
            TC_REQUIRE(reinterpret_cast<uintptr_t>(indexed->cache_batch_idx) % 4 == 0, "misaligned cache_batch_idx");
        }
    }
    const size_t q_bytes = size_t(rows) * kDim * 2, cache_bytes = size_t(cache_slots) * slot_rows * kv_heads * kDim * 2;
    const size_t new_bytes = size_t(batch) * kv_heads * kDim * 2;
    TC_REQUIRE(cache_bytes <= (size_t(1) << 40), "cache allocation is outside the supported range");
    const int64_t need_o = splits > 1 ? int64_t(splits) * rows * kDim : 0, need_lse = splits > 1 ? int64_t(splits) * rows : 0;
    TC_REQUIRE(workspace_o_elems >= need_o && workspace_lse_elems >= need_lse,
               "Preallocated complete split workspace is too small");
    TC_REQUIRE(!need_o || (workspace_o && workspace_lse), "null split workspace");
    const void* pointers[10] = {q, kcache, vcache, knew, vnew, old_lengths, partial == 1 ? (void*)partial_o : out, lse,
                                need_o ? workspace_o : nullptr, need_lse ? workspace_lse : nullptr};
    const size_t sizes[10] = {q_bytes, cache_bytes, cache_bytes, new_bytes, new_bytes, size_t(batch) * 4,
                              partial == 1 ? size_t(rows) * kDim * 4 : q_bytes, size_t(rows) * 4, size_t(need_o) * 4,
                              size_t(need_lse) * 4};
    for (int i = 0; i < 10; ++i)
        for (int j = i + 1; j < 10; ++j)
            TC_REQUIRE(!pointers[i] || !pointers[j] || !tc::ranges_overlap(pointers[i], sizes[i], pointers[j], sizes[j]),
                       "All nonempty ABI tensor allocations must be disjoint");
    for (int i = 0; i < 10; ++i)
        TC_REQUIRE(!pointers[i] || reinterpret_cast<uintptr_t>(pointers[i]) % 16 == 0 || i == 5 || i == 7,
                   "16-byte aligned storage required");
    TC_REQUIRE(reinterpret_cast<uintptr_t>(old_lengths) % 4 == 0 && reinterpret_cast<uintptr_t>(lse) % 4 == 0,
               "misaligned old_lengths or LSE");

    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    tc::DeviceScratch scratch;
    status = tc::device_scratch(device, &scratch);
    if (status != TC_OK) return status;
    CUtensorMap kmap, vmap;
    status = cache_map(device, kcache, cache_slots, slot_rows, kv_heads, &kmap);
    if (status != TC_OK) return status;
    status = cache_map(device, vcache, cache_slots, slot_rows, kv_heads, &vmap);
    if (status != TC_OK) return status;

    DecodeParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.kcache = static_cast<__nv_bfloat16*>(kcache);
    p.vcache = static_cast<__nv_bfloat16*>(vcache);
    p.knew = static_cast<const __nv_bfloat16*>(knew);
    p.vnew = static_cast<const __nv_bfloat16*>(vnew);
    p.old_lengths = old_lengths;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.lse = lse;
    p.partial_o = partial_o;
    p.page_size = int(slot_rows);
    p.cache_slots = int(cache_slots);
    p.cache_stable = cache_stable;
    if (rope) {
        TC_REQUIRE(rope->cos && rope->sin && rope->positions >= 1 && rope->positions <= (int64_t(1) << 30),
                   "RoPE needs cos/sin tables FP32[positions,64] with positions >= 1");
        TC_REQUIRE(reinterpret_cast<uintptr_t>(rope->cos) % 16 == 0 && reinterpret_cast<uintptr_t>(rope->sin) % 16 == 0,
                   "16-byte aligned RoPE tables required");
        p.rope_cos = rope->cos;
        p.rope_sin = rope->sin;
        p.rope_positions = int(rope->positions);
    }
    if (indexed) {
        p.block_table = indexed->block_table;
        p.table_stride = indexed->table_stride;
        p.cache_batch_idx = indexed->cache_batch_idx;
    }
    p.ws_o = workspace_o;
    p.ws_lse = workspace_lse;
    p.tickets = scratch.tickets;
    p.status = scratch.status;
    p.batch = int(batch);
    p.capacity = int(capacity);
    p.kv_heads = int(kv_heads);
    p.splits = splits;
    p.append = append ? 1 : 0;
    p.partial = partial;
    p.shard_start = shard_start;
    p.scale = 1.f / std::sqrt(128.f);
    p.scale_log2 = p.scale * float(M_LOG2E);
    if (peer) {
        p.world = peer->world;
        p.rank = peer->rank;
        for (int r = 0; r < peer->world; ++r) p.peer_blocks[r] = static_cast<uint8_t*>(peer->blocks[r]);
        return mapping == 1 ? launch<true, true>(kmap, vmap, p, static_cast<cudaStream_t>(stream))
                            : launch<false, true>(kmap, vmap, p, static_cast<cudaStream_t>(stream));
    }
    return mapping == 1 ? launch<true>(kmap, vmap, p, static_cast<cudaStream_t>(stream))
                        : launch<false>(kmap, vmap, p, static_cast<cudaStream_t>(stream));
}


// ------------------------------------------------------------------------------- allocation-free variant
// Scratch for tc_decode_forward_out_static: split partials, split tickets and a status word in one
// file-scope device array, so the call never allocates. In host code the array's name is only a
// stand-in for the symbol; the device address comes from cudaGetSymbolAddress (once per device).
constexpr int kStaticMaxRows = 128;    // batch * query heads (e.g. batch 4 x 32 heads)
constexpr int kStaticMaxSplits = 32;
constexpr size_t kStaticOFloats = size_t(kStaticMaxSplits) * kStaticMaxRows * kDim;
constexpr size_t kStaticLseFloats = size_t(kStaticMaxSplits) * kStaticMaxRows;
constexpr size_t kStaticTicketWords = kStaticMaxRows / kGroup;
constexpr size_t kStaticStatusWord = kStaticOFloats + kStaticLseFloats + kStaticTicketWords;
constexpr size_t kStaticWords = kStaticStatusWord + 64;
static __device__ __align__(256) float g_static_scratch[kStaticWords];  // 2.1 MiB per GPU that loads the library

int static_scratch_address(int device, float** address) {
    static std::mutex lock;
    static std::unordered_map<int, float*> known;
    std::lock_guard<std::mutex> guard(lock);
    auto found = known.find(device);
    if (found == known.end()) {
        void* pointer = nullptr;  // `device` is current here: the caller holds a DeviceGuard
        TC_CUDA(cudaGetSymbolAddress(&pointer, g_static_scratch));
        TC_REQUIRE(pointer != nullptr, "cudaGetSymbolAddress returned a null scratch address");
        found = known.emplace(device, static_cast<float*>(pointer)).first;
        // The kernel status word of static calls lives in the array too: tell tc_device_status where.
        tc::register_status_word(device, reinterpret_cast<int32_t*>(found->second + kStaticStatusWord));
    }
    *address = found->second;
    return TC_OK;
}

int decode_static(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                  const void* vnew, const int32_t* old_lengths, void* out, float* lse, int64_t batch,
                  int64_t capacity, int64_t kv_heads, int64_t num_splits, int64_t mapping, int append) {
    tc::DeviceInfo info;
    int splits = 1;
    int status = check_geometry(device, batch, capacity, kv_heads, num_splits, mapping, append, &info, &splits);
    if (status != TC_OK) return status;
    TC_REQUIRE(q && kcache && vcache && knew && vnew && old_lengths && lse && out, "null tensor pointer");
    const int64_t rows = batch * kv_heads * kGroup;
    TC_REQUIRE(rows <= kStaticMaxRows,
               "tc_decode_forward_out_static: batch * query heads = %lld exceeds the built-in scratch (max %d rows); "
               "use tc_decode_forward_out with a caller workspace", static_cast<long long>(rows), kStaticMaxRows);
    if (num_splits == 0 && splits > kStaticMaxSplits) splits = kStaticMaxSplits;
    TC_REQUIRE(splits <= kStaticMaxSplits,
               "tc_decode_forward_out_static: %d splits exceed the built-in scratch (max %d)", splits, kStaticMaxSplits);
    const size_t q_bytes = size_t(rows) * kDim * 2, cache_bytes = size_t(batch) * capacity * kv_heads * kDim * 2;
    const size_t new_bytes = size_t(batch) * kv_heads * kDim * 2;
    const void* pointers[8] = {q, kcache, vcache, knew, vnew, old_lengths, out, lse};
    const size_t sizes[8] = {q_bytes, cache_bytes, cache_bytes, new_bytes, new_bytes, size_t(batch) * 4, q_bytes,
                             size_t(rows) * 4};
    for (int i = 0; i < 8; ++i)
        for (int j = i + 1; j < 8; ++j)
            TC_REQUIRE(!tc::ranges_overlap(pointers[i], sizes[i], pointers[j], sizes[j]),
                       "All nonempty ABI tensor allocations must be disjoint");
    for (int i = 0; i < 7; ++i)
        TC_REQUIRE(reinterpret_cast<uintptr_t>(pointers[i]) % 16 == 0 || i == 5, "16-byte aligned storage required");
    TC_REQUIRE(reinterpret_cast<uintptr_t>(old_lengths) % 4 == 0 && reinterpret_cast<uintptr_t>(lse) % 4 == 0,
               "misaligned old_lengths or LSE");

    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    float* scratch = nullptr;
    if ((status = static_scratch_address(device, &scratch)) != TC_OK) return status;
    int32_t* tickets = reinterpret_cast<int32_t*>(scratch + kStaticOFloats + kStaticLseFloats);
    CUtensorMap kmap, vmap;  // encoded on the stack: this path keeps no host-side cache either
    if ((status = tc::make_rows_map(&kmap, kcache, false, kv_heads, capacity, batch, kDim, kv_heads * kDim,
                                    capacity * kv_heads * kDim, kTileN, 2)) != TC_OK) return status;
    if ((status = tc::make_rows_map(&vmap, vcache, false, kv_heads, capacity, batch, kDim, kv_heads * kDim,
                                    capacity * kv_heads * kDim, kTileN, 2)) != TC_OK) return status;
    // The tickets must start at zero; the kernel leaves them at zero, but a launch that was cut short
    // must not poison the next one, so they are cleared on the stream every time. The status word next
    // to them is NOT cleared here: it keeps the first non-zero code until tc_device_status reads it.
    TC_CUDA(cudaMemsetAsync(tickets, 0, kStaticTicketWords * sizeof(int32_t), static_cast<cudaStream_t>(stream)));

    DecodeParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.kcache = static_cast<__nv_bfloat16*>(kcache);
    p.vcache = static_cast<__nv_bfloat16*>(vcache);
    p.knew = static_cast<const __nv_bfloat16*>(knew);
    p.vnew = static_cast<const __nv_bfloat16*>(vnew);
    p.old_lengths = old_lengths;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.lse = lse;
    p.partial_o = nullptr;
    p.ws_o = scratch;
    p.ws_lse = scratch + kStaticOFloats;
    p.tickets = tickets;
    p.status = reinterpret_cast<int32_t*>(scratch + kStaticStatusWord);
    p.batch = int(batch);
    p.capacity = int(capacity);
    p.kv_heads = int(kv_heads);
    p.splits = splits;
    p.append = append ? 1 : 0;
    p.partial = 0;
    p.shard_start = 0;
    p.page_size = int(capacity);
    p.cache_slots = int(batch);
    p.scale = 1.f / std::sqrt(128.f);
    p.scale_log2 = p.scale * float(M_LOG2E);
    return mapping == 1 ? launch<true>(kmap, vmap, p, static_cast<cudaStream_t>(stream))
                        : launch<false>(kmap, vmap, p, static_cast<cudaStream_t>(stream));
}

}  // namespace

extern "C" {

int tc_decode_workspace_spec(int device, int64_t batch, int64_t capacity, int64_t kv_heads, int64_t num_splits,
                             int64_t mapping, int append, int64_t spec[3]) {
    tc::DeviceInfo info;
    int splits = 1;
    int status = check_geometry(device, batch, capacity, kv_heads, num_splits, mapping, append, &info, &splits);
    if (status != TC_OK) return status;
    TC_REQUIRE(spec, "null spec");
    const int64_t rows = batch * kv_heads * kGroup;
    spec[0] = splits;
    spec[1] = splits > 1 ? splits * rows * kDim : 0;
    spec[2] = splits > 1 ? splits * rows : 0;
    return TC_OK;
}

int tc_decode_forward_out(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                          const void* vnew, const int32_t* old_lengths, void* out, float* lse, float* workspace_o,
                          int64_t workspace_o_elems, float* workspace_lse, int64_t workspace_lse_elems, int64_t batch,
                          int64_t capacity, int64_t kv_heads, int64_t num_splits, int64_t mapping, int append) {
    return decode_common(device, stream, q, kcache, vcache, knew, vnew, old_lengths, out, lse, nullptr, workspace_o,
                         workspace_o_elems, workspace_lse, workspace_lse_elems, batch, capacity, kv_heads, num_splits,
                         mapping, append, 0, 0);
}

int tc_decode_partial_out(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                          const void* vnew, const int32_t* old_lengths, float* partial_o, float* partial_lse,
                          float* workspace_o, int64_t workspace_o_elems, float* workspace_lse,
                          int64_t workspace_lse_elems, int64_t batch, int64_t capacity, int64_t kv_heads,
                          int64_t num_splits, int64_t mapping, int append, int64_t kv_shard_start) {
    return decode_common(device, stream, q, kcache, vcache, knew, vnew, old_lengths, nullptr, partial_lse, partial_o,
                         workspace_o, workspace_o_elems, workspace_lse, workspace_lse_elems, batch, capacity, kv_heads,
                         num_splits, mapping, append, 1, kv_shard_start);
}

int tc_combine_partials(int device, void* stream, const float* partial_o, const float* partial_lse, int64_t parts,
                        int64_t rows, int64_t part_stride_o, int64_t part_stride_lse, void* out, float* lse) {
    tc::DeviceInfo info;
    int status = tc::require_sm100(device, &info);
    if (status != TC_OK) return status;
    TC_REQUIRE(partial_o && partial_lse && out && lse, "null tensor pointer");
    TC_REQUIRE(parts >= 1 && parts <= 1024 && rows >= 1 && rows <= (int64_t(1) << 24), "parts or rows out of range");
    TC_REQUIRE(reinterpret_cast<uintptr_t>(partial_o) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 8 == 0 &&
                   part_stride_o % 4 == 0,
               "16-byte aligned partial O (base and part stride) and 8-byte aligned O required");
    TC_REQUIRE(part_stride_o >= rows * kDim && part_stride_lse >= rows, "part strides smaller than one part");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    const unsigned blocks = unsigned((rows + 3) / 4);
    combine_partials_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        partial_o, partial_lse, int(parts), rows, part_stride_o, part_stride_lse, static_cast<__nv_bfloat16*>(out), lse);
    TC_CUDA(cudaGetLastError());
    return TC_OK;
}

int tc_decode_resources(int device, int64_t batch, int64_t capacity, int64_t kv_heads, int64_t num_splits,
                        int64_t mapping, int append, int64_t* values, int64_t capacity_values, int64_t* count) {
    tc::DeviceInfo info;
    int splits = 1;
    int status = check_geometry(device, batch, capacity, kv_heads, num_splits, mapping, append, &info, &splits);
    if (status != TC_OK) return status;
    TC_REQUIRE(append, "Resource reporting requires fused KV append");
    TC_REQUIRE(values && count && capacity_values >= 34, "resources needs room for 34 values");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    const int64_t rows = batch * kv_heads * kGroup;
    const int64_t header[12] = {splits, kGroup, kv_heads, kGroup, 1, batch * kv_heads * splits,
                                splits > 1 ? batch * kv_heads : 0, splits > 1 ? splits * rows * kDim : 0,
                                splits > 1 ? splits * rows : 0, kGroup, kTileN, 1};
    for (int i = 0; i < 12; ++i) values[i] = header[i];
    status = mapping == 1 ? tc::kernel_resources(&decode_splitkv_kernel<true, false>, kThreads, shared_bytes(true), values + 12)
                          : tc::kernel_resources(&decode_splitkv_kernel<false, false>, kThreads, shared_bytes(false), values + 12);
    if (status != TC_OK) return status;
    status = tc::kernel_resources(&combine_partials_kernel, 128, 0, values + 20);
    if (status != TC_OK) return status;
    const int64_t tail[6] = {capacity, capacity - 1, capacity - 1 + (append ? 1 : 0), append ? 1 : 0, mapping == 0,
                             V10_FAMILY_CODE};
    for (int i = 0; i < 6; ++i) values[28 + i] = tail[i];
    *count = 34;
    return TC_OK;
}

int tc_decode_forward_out_static(int device, void* stream, const void* q, void* kcache, void* vcache,
                                 const void* knew, const void* vnew, const int32_t* old_lengths, void* out,
                                 float* lse, int64_t batch, int64_t capacity, int64_t kv_heads, int64_t num_splits,
                                 int64_t mapping, int append) {
    return decode_static(device, stream, q, kcache, vcache, knew, vnew, old_lengths, out, lse, batch, capacity,
                         kv_heads, num_splits, mapping, append);
}

#ifdef TC_TRACE
// Trace builds only: copies the 1024 x 32 table of time stamps to `host` (synchronises the device).
int tc_debug_trace(void* host) { return cudaMemcpyFromSymbol(host, g_trace, sizeof(g_trace)) == cudaSuccess ? 0 : 1; }
#endif

int tc_decode_static_status_word(int device, int32_t** word) {
    TC_REQUIRE(word, "null output");
    tc::DeviceInfo info;
    int status = tc::require_sm100(device, &info);
    if (status != TC_OK) return status;
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    float* scratch = nullptr;
    if ((status = static_scratch_address(device, &scratch)) != TC_OK) return status;
    *word = reinterpret_cast<int32_t*>(scratch + kStaticStatusWord);
    return TC_OK;
}

int tc_decode_indexed_forward_out(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                                  const void* vnew, const int32_t* old_lengths, void* out, float* lse,
                                  float* workspace_o, int64_t workspace_o_elems, float* workspace_lse,
                                  int64_t workspace_lse_elems, int64_t batch, int64_t cache_slots, int64_t slot_rows,
                                  int64_t kv_heads, int64_t num_splits, int64_t mapping, int append,
                                  const int32_t* block_table, int64_t block_table_stride, int64_t pages_per_seq,
                                  const int32_t* cache_batch_idx) {
    TC_REQUIRE(block_table || cache_batch_idx, "pass a block table or cache_batch_idx (or use tc_decode_forward_out)");
    TC_REQUIRE(slot_rows >= 1 && pages_per_seq >= 0 && pages_per_seq <= (int64_t(1) << 24), "geometry out of range");
    const IndexedCache indexed{block_table, block_table_stride, pages_per_seq, cache_batch_idx, cache_slots, slot_rows};
    const int64_t capacity = block_table ? pages_per_seq * slot_rows : slot_rows;
    return decode_common(device, stream, q, kcache, vcache, knew, vnew, old_lengths, out, lse, nullptr, workspace_o,
                         workspace_o_elems, workspace_lse, workspace_lse_elems, batch, capacity, kv_heads, num_splits,
                         mapping, append, 0, 0, nullptr, &indexed);
}

int tc_decode_rope_forward_out(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                               const void* vnew, const int32_t* old_lengths, void* out, float* lse, float* workspace_o,
                               int64_t workspace_o_elems, float* workspace_lse, int64_t workspace_lse_elems,
                               int64_t batch, int64_t capacity, int64_t kv_heads, int64_t num_splits, int64_t mapping,
                               int append, const float* rope_cos, const float* rope_sin, int64_t rope_positions) {
    const RopeTables rope{rope_cos, rope_sin, rope_positions};
    return decode_common(device, stream, q, kcache, vcache, knew, vnew, old_lengths, out, lse, nullptr, workspace_o,
                         workspace_o_elems, workspace_lse, workspace_lse_elems, batch, capacity, kv_heads, num_splits,
                         mapping, append, 0, 0, nullptr, nullptr, &rope);
}

int tc_decode_forward_out_flags(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                                const void* vnew, const int32_t* old_lengths, void* out, float* lse,
                                float* workspace_o, int64_t workspace_o_elems, float* workspace_lse,
                                int64_t workspace_lse_elems, int64_t batch, int64_t capacity, int64_t kv_heads,
                                int64_t num_splits, int64_t mapping, int append, int64_t flags) {
    TC_REQUIRE((flags & ~int64_t(TC_DECODE_CACHE_STABLE | TC_DECODE_PREFIX_STABLE)) == 0, "unknown decode flag");
    TC_REQUIRE(flags != (TC_DECODE_CACHE_STABLE | TC_DECODE_PREFIX_STABLE),
               "TC_DECODE_CACHE_STABLE and TC_DECODE_PREFIX_STABLE are alternatives");
    return decode_common(device, stream, q, kcache, vcache, knew, vnew, old_lengths, out, lse, nullptr, workspace_o,
                         workspace_o_elems, workspace_lse, workspace_lse_elems, batch, capacity, kv_heads, num_splits,
                         mapping, append, 0, 0, nullptr, nullptr, nullptr,
                         (flags & TC_DECODE_CACHE_STABLE) ? 1 : ((flags & TC_DECODE_PREFIX_STABLE) ? 2 : 0));
}

int tc_peer_block_bytes(int64_t batch, int64_t kv_heads, int64_t world, int64_t* bytes) {
    TC_REQUIRE(bytes, "null bytes");
    TC_REQUIRE(batch >= 1 && batch <= 65535 && kv_heads >= 1 && kv_heads <= 8 && world >= 1 && world <= kMaxPeers,
               "peer exchange needs 1 <= B <= 65535, 1 <= Hkv <= 8, 1 <= world <= 8");
    *bytes = int64_t(peer_block_bytes(int(world), int(batch * kv_heads)));
    return TC_OK;
}

int tc_peer_block_create(int device, int64_t bytes, void** block, unsigned char* handle64) {
    TC_REQUIRE(block && handle64 && bytes > 0, "null output or empty block");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    void* pointer = nullptr;
    TC_CUDA(cudaMalloc(&pointer, size_t(bytes)));
    cudaError_t error = cudaMemset(pointer, 0, size_t(bytes));  // flags and epochs start at zero
    cudaIpcMemHandle_t handle;
    if (error == cudaSuccess) error = cudaIpcGetMemHandle(&handle, pointer);
    if (error != cudaSuccess) {
        cudaFree(pointer);
        TC_CUDA(error);
    }
    std::memcpy(handle64, &handle, 64);
    *block = pointer;
    return TC_OK;
}

int tc_peer_block_open(int device, const unsigned char* handle64, void** block) {
    TC_REQUIRE(block && handle64, "null handle or output");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    cudaIpcMemHandle_t handle;
    std::memcpy(&handle, handle64, 64);
    TC_CUDA(cudaIpcOpenMemHandle(block, handle, cudaIpcMemLazyEnablePeerAccess));
    return TC_OK;
}

int tc_peer_block_close(int device, void* block) {
    TC_REQUIRE(block, "null block");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    TC_CUDA(cudaIpcCloseMemHandle(block));
    return TC_OK;
}

int tc_peer_block_destroy(int device, void* block) {
    TC_REQUIRE(block, "null block");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    TC_CUDA(cudaFree(block));
    return TC_OK;
}

int tc_decode_exchange_out(int device, void* stream, const void* q, void* kcache, void* vcache, const void* knew,
                           const void* vnew, const int32_t* old_lengths, void* out, float* lse, float* workspace_o,
                           int64_t workspace_o_elems, float* workspace_lse, int64_t workspace_lse_elems, int64_t batch,
                           int64_t capacity, int64_t kv_heads, int64_t num_splits, int64_t mapping, int append,
                           int64_t kv_shard_start, int64_t world, int64_t rank, void* const* peer_blocks,
                           int64_t peer_block_size) {
    TC_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, "need 1 <= world <= 8, 0 <= rank < world");
    // The kernel derives every slot and epoch offset from (batch, kv_heads, world) and stores into every
    // rank's block: a block made for a smaller geometry would take stores past its end, on another GPU.
    TC_REQUIRE(batch >= 1 && batch <= 65535 && kv_heads >= 1 && kv_heads <= 8, "batch or kv_heads out of range");
    TC_REQUIRE(peer_block_size >= int64_t(peer_block_bytes(int(world), int(batch * kv_heads))),
               "exchange blocks of %lld bytes are too small for batch %lld, %lld KV heads, %lld ranks (need %lld)",
               static_cast<long long>(peer_block_size), static_cast<long long>(batch),
               static_cast<long long>(kv_heads), static_cast<long long>(world),
               static_cast<long long>(peer_block_bytes(int(world), int(batch * kv_heads))));
    const PeerArgs peer{peer_blocks, int(world), int(rank)};
    return decode_common(device, stream, q, kcache, vcache, knew, vnew, old_lengths, out, lse, nullptr, workspace_o,
                         workspace_o_elems, workspace_lse, workspace_lse_elems, batch, capacity, kv_heads, num_splits,
                         mapping, append, 2, kv_shard_start, &peer);
}

}  // extern "C"
