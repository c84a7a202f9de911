// The step before decode attention, for one new token per sequence: fused QKV projection, per-head
// RMS normalisation of q and k (Qwen3 style, optional), rotary position embedding of q and k, and
// output in exactly the layout the decode kernel consumes (q [B,1,Hq,128], knew / vnew [B,1,Hkv,128]).
//
// The reference stops short of this step: its decode kernel is handed "pre-rotated Q/K ... and one
// new row" (tilecadence/cuda/decode/ab_fused_splitkv.cuh:189) computed elsewhere. This file has no
// counterpart there.
//
// y = x W^T with x [tokens <= 8, hidden] and W [(Hq + 2 Hkv) * 128, hidden] (BF16, row-major, q heads
// first, then k heads, then v heads) is a weight-streaming problem: every weight byte is read once
// (31.5 MB for hidden 2560, 32 + 8 + 8 heads), the arithmetic is negligible, so the bound is HBM
// bandwidth. One cluster of `splits` CTAs owns one head's 128 output rows; CTA r of the cluster
// streams the r-th slice of the hidden dimension as 128-row x 64-column weight tiles (16 KiB, TMA,
// 128-byte swizzle, 5-stage mbarrier ring), multiplies with warp-level BF16 MMAs against the token slab held in
// shared memory, and ships its 128 x 8 partial sums into CTA 0's shared memory (distributed shared
// memory stores + one cluster barrier). CTA 0 finishes the head: sum, RMS norm, RoPE, BF16 stores.
#include "tc_host.cuh"
#include "tc_ptx.cuh"

#include <cmath>

namespace {

constexpr int kRows = 128;                       // outputs of one head
constexpr int kTileK = 64;                       // hidden elements per weight tile: 128-byte rows
constexpr int kTileBytes = kRows * kTileK * 2;   // 16 KiB
constexpr int kStages = 5;                       // 80 KiB ring: two CTAs fit one SM at hidden 2560, so the next
                                                 // launch's CTAs can start their weight ring during this one's tail
constexpr int kWarps = 8;                        // 16 output rows per consumer warp
constexpr int kConsumerThreads = kWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + one TMA producer warp
constexpr int kMaxTokens = 8;                    // the MMA's n
constexpr int kMaxSplits = 4;
constexpr int kMaxHidden = 16384;

struct ProjectParams {
    const __nv_bfloat16* x;         // [tokens, hidden]
    const __nv_bfloat16* q_norm;    // [128] or nullptr
    const __nv_bfloat16* k_norm;    // [128] or nullptr
    const float* rope_cos;          // [rope_positions, 64] or nullptr
    const float* rope_sin;
    const int32_t* positions;       // [tokens]
    __nv_bfloat16* q_out;           // [tokens, q_heads, 128]
    __nv_bfloat16* k_out;           // [tokens, kv_heads, 128]
    __nv_bfloat16* v_out;
    int32_t* status;
    int tokens, hidden, q_heads, kv_heads, splits, rope_positions;
    int release_early;              // TC_PROJECT_RELEASE_EARLY: dependents may be scheduled before this launch's own wait
    float eps;
};

// Shared-memory plan (bytes from a 1024-aligned base): weight ring | token slab | partials received
// from the other CTAs of the cluster | this head's sums | barriers.
__host__ __device__ constexpr int slab_row_bytes(int k_local) { return k_local * 2 + 16; }  // +16: no bank conflicts
__host__ __device__ constexpr int slab_offset() { return kStages * kTileBytes; }
__host__ __device__ constexpr int recv_offset(int k_local) { return slab_offset() + (kMaxTokens * slab_row_bytes(k_local) + 127) / 128 * 128; }
__host__ __device__ constexpr int sums_offset(int k_local) { return recv_offset(k_local) + (kMaxSplits - 1) * kRows * kMaxTokens * 4; }
__host__ __device__ constexpr int barrier_offset(int k_local) { return sums_offset(k_local) + kRows * kMaxTokens * 4; }
__host__ __device__ constexpr int shared_bytes(int k_local) { return 1024 + barrier_offset(k_local) + 128; }

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Build switch TC_TRACE (off in every shipped library): thread 0 and the producer lane of every CTA record
// %globaltimer at the points below into a device table that tc_debug_project_trace copies out; see
// tilecadence_b200/trace_project.py.
//   0 entry  1 ring and L2 prefetch issued  2 stream dependency resolved  3 token slab ready  4 tile 0 arrived
//   5 first refilled tile arrived  6 weight loop done  7 cluster barrier passed  8 head stored (rank 0)
#ifdef TC_TRACE
__device__ unsigned long long g_project_trace[256][16];
#define TC_TRACE_POINT(slot) do { if (trace_row) trace_row[slot] = tc::global_timer_ns(); } while (0)
#else
#define TC_TRACE_POINT(slot) do { } while (0)
#endif

__global__ void __launch_bounds__(kThreads, 2)
qkv_rope_kernel(const __grid_constant__ CUtensorMap wmap, const ProjectParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = int(tc::cluster_cta_rank());
    const int head = blockIdx.y;
#ifdef TC_TRACE
    unsigned long long* trace_row = (threadIdx.x == 0 || threadIdx.x == kWarps * 32)
                                        ? g_project_trace[(blockIdx.y * gridDim.x + blockIdx.x) & 255] : nullptr;
#endif
    if (threadIdx.x == 0) TC_TRACE_POINT(0);

    const int tiles_total = p.hidden / kTileK;
    const int tile_begin = rank * tiles_total / p.splits, tile_end = (rank + 1) * tiles_total / p.splits;
    const int n_tiles = tile_end - tile_begin;
    const int k_local_max = ((tiles_total + p.splits - 1) / p.splits) * kTileK;  // same plan in every CTA of the cluster
    const int row_bytes = slab_row_bytes(k_local_max);
    uint8_t* slab = smem + slab_offset();
    float* recv = reinterpret_cast<float*>(smem + recv_offset(k_local_max));
    float* sums = reinterpret_cast<float*>(smem + sums_offset(k_local_max));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + barrier_offset(k_local_max));
    uint64_t* empty = full + kStages;

    // The producer sets up the ring and sends for the first stages at once: the weights do not depend
    // on anything the preceding kernel in the stream produced, so with programmatic dependent launch this
    // part overlaps that kernel's tail; x, the positions and the outputs are touched only after the wait.
    const uint64_t policy = tc::policy_evict_first();
    auto load_tile = [&](int it) {
        const int stage = it % kStages;
        tc::mbar_arrive_expect_tx(&full[stage], kTileBytes);
        tc::tma_load_2d(smem + stage * kTileBytes, &wmap, &full[stage], (tile_begin + it) * kTileK, head * kRows, policy);
    };
    if (threadIdx.x == kWarps * 32) {
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], kWarps);
        }
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&wmap);
        for (int it = 0; it < kStages && it < n_tiles; ++it) load_tile(it);
        // The rest of this CTA's weight slice is asked into L2 behind the ring: the stream from HBM then runs
        // through the preceding kernel's tail instead of stopping when the ring is full, and after the wait the
        // ring refills from L2.
        for (int it = kStages; it < n_tiles; ++it) tc::tma_prefetch_2d(&wmap, (tile_begin + it) * kTileK, head * kRows);
        TC_TRACE_POINT(1);
    }
    // By default the launch that follows is released once this one has seen its own dependency resolve, so that it
    // overlaps this launch only. With the caller's promise that the follower's independent part is also safe beside
    // the kernel BEFORE this one, it is released at once: its CTAs then take the SM slots as that kernel's CTAs leave
    // them, a few microseconds earlier, and its weight stream starts that much sooner.
    if (p.release_early) tc::grid_launch_dependents();
    tc::grid_dependency_wait();
    if (threadIdx.x == 0) TC_TRACE_POINT(2);
    if (!p.release_early) tc::grid_launch_dependents();
    // Token slab: this CTA's slice of every token's hidden vector, zero rows for absent tokens.
    {
        const int chunks = n_tiles * kTileK / 8;  // 16-byte chunks per token
        for (int idx = threadIdx.x; idx < kMaxTokens * chunks; idx += kThreads) {
            const int n = idx / chunks, c = idx - n * chunks;
            uint4 value = make_uint4(0, 0, 0, 0);
            if (n < p.tokens)
                value = __ldg(reinterpret_cast<const uint4*>(p.x + int64_t(n) * p.hidden + tile_begin * kTileK) + c);
            *reinterpret_cast<uint4*>(slab + n * row_bytes + c * 16) = value;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) TC_TRACE_POINT(3);

    // Rank 0 finishes the head with one warp per token: what that needs from global memory (norm weights, the
    // token's position and its rotary table rows: two dependent loads) is sent for now and arrives during the
    // weight loop instead of after the cluster barrier.
    const bool is_q = head < p.q_heads, is_k = !is_q && head < p.q_heads + p.kv_heads;
    const __nv_bfloat16* norm = is_q ? p.q_norm : (is_k ? p.k_norm : nullptr);
    const bool rotates = p.rope_cos && (is_q || is_k);
    float norm_weight[4] = {1.f, 1.f, 1.f, 1.f}, rope_c[2] = {1.f, 1.f}, rope_s[2] = {0.f, 0.f};
    if (rank == 0 && warp < p.tokens) {
        if (norm) {
#pragma unroll
            for (int j = 0; j < 4; ++j) norm_weight[j] = __bfloat162float(norm[lane + 32 * j]);
        }
        if (rotates) {
            int position = p.positions[warp];
            position = position < 0 ? 0 : (position >= p.rope_positions ? p.rope_positions - 1 : position);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                rope_c[j] = p.rope_cos[int64_t(position) * 64 + lane + 32 * j];
                rope_s[j] = p.rope_sin[int64_t(position) * 64 + lane + 32 * j];
            }
        }
    }

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    bool failed = false;
    if (warp == kWarps) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int it = kStages; it < n_tiles; ++it) {
                if (!tc::mbar_wait(&empty[it % kStages], (uint32_t(it / kStages) & 1) ^ 1)) {
                    atomicCAS(p.status, 0, 21);
                    break;
                }
                load_tile(it);
            }
        }
    } else {
        // ------------------------------------------------------------------ consumers: 16 rows per warp
        const uint32_t slab_addr = tc::smem_u32(slab);
        const uint32_t a_row = uint32_t(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8);  // ldmatrix row of this lane
        const uint32_t a_half = uint32_t(lane >> 4);                                        // k 0-7 or 8-15
        const uint32_t b_lane = slab_addr + uint32_t(lane & 7) * row_bytes + uint32_t((lane >> 3) & 1) * 16;
        for (int it = 0; it < n_tiles; ++it) {
            const int stage = it % kStages;
            if (!tc::mbar_wait(&full[stage], uint32_t(it / kStages) & 1)) {
                failed = true;
                break;
            }
            if (threadIdx.x == 0 && it == 0) TC_TRACE_POINT(4);
            if (threadIdx.x == 0 && it == kStages) TC_TRACE_POINT(5);
            const uint32_t tile = tc::smem_u32(smem + stage * kTileBytes);
#pragma unroll
            for (int ks = 0; ks < kTileK / 16; ++ks) {
                const uint32_t chunk = uint32_t(ks * 2) + a_half;
                uint32_t a0, a1, a2, a3, b0, b1;
                tc::ldmatrix_x4(tile + a_row * 128 + ((chunk ^ (a_row & 7)) << 4), a0, a1, a2, a3);
                tc::ldmatrix_x2(b_lane + uint32_t(it * kTileK + ks * 16) * 2, b0, b1);
                tc::mma_bf16_16816(acc, a0, a1, a2, a3, b0, b1);
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&empty[stage]);
        }
        if (failed) atomicCAS(p.status, 0, 22);
        if (threadIdx.x == 0) TC_TRACE_POINT(6);
        // Partial sums of rows g, g + 8 (of this warp's 16) for tokens 2t, 2t + 1.
        const int g = lane >> 2, t = lane & 3;
        const int row0 = warp * 16 + g;
        float* target = rank == 0 ? sums : recv + (rank - 1) * kRows * kMaxTokens;
        if (rank == 0) {
            *reinterpret_cast<float2*>(target + row0 * kMaxTokens + 2 * t) = make_float2(acc[0], acc[1]);
            *reinterpret_cast<float2*>(target + (row0 + 8) * kMaxTokens + 2 * t) = make_float2(acc[2], acc[3]);
        } else {
            tc::cluster_store_f32x2(tc::cluster_map_shared(target + row0 * kMaxTokens + 2 * t, 0), acc[0], acc[1]);
            tc::cluster_store_f32x2(tc::cluster_map_shared(target + (row0 + 8) * kMaxTokens + 2 * t, 0), acc[2], acc[3]);
        }
    }
    // Every thread of every CTA of the cluster arrives here (nobody has exited): the partials of
    // ranks > 0 are in rank 0's shared memory afterwards.
    __syncwarp();
    tc::cluster_sync();
    if (threadIdx.x == 0) TC_TRACE_POINT(7);
    if (rank != 0 || warp == kWarps) return;

    // ---------------------------------------------------------------------- finish the head (rank 0)
    for (int idx = threadIdx.x; idx < kRows * kMaxTokens; idx += kConsumerThreads) {
        float total = sums[idx];
        for (int r = 1; r < p.splits; ++r) total += recv[(r - 1) * kRows * kMaxTokens + idx];
        sums[idx] = total;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
    const int token = warp;  // one warp per token
    if (token >= p.tokens) return;
    // Lane l owns outputs l, l + 32, l + 64, l + 96: both RoPE pairs (i, i + 64) stay in the thread.
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = sums[(lane + 32 * j) * kMaxTokens + token];
    if (norm) {
        // RMS norm as Qwen3 applies it per head: x * rsqrt(mean(x^2) + eps) rounded to BF16, times the
        // BF16 weight, rounded to BF16.
        float square = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) square += __shfl_xor_sync(0xffffffffu, square, offset);
        const float inv = rsqrtf(square * (1.f / kRows) + p.eps);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            v[j] = round_bf16(round_bf16(v[j] * inv) * norm_weight[j]);
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = round_bf16(v[j]);
    }
    if (rotates) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float cs = rope_c[j], sn = rope_s[j];
            const float lo = __fsub_rn(__fmul_rn(v[j], cs), __fmul_rn(v[j + 2], sn));
            const float hi = __fadd_rn(__fmul_rn(v[j + 2], cs), __fmul_rn(v[j], sn));
            v[j] = lo;
            v[j + 2] = hi;
        }
    }
    __nv_bfloat16* out = is_q   ? p.q_out + (int64_t(token) * p.q_heads + head) * kRows
                         : is_k ? p.k_out + (int64_t(token) * p.kv_heads + (head - p.q_heads)) * kRows
                                : p.v_out + (int64_t(token) * p.kv_heads + (head - p.q_heads - p.kv_heads)) * kRows;
#pragma unroll
    for (int j = 0; j < 4; ++j) out[lane + 32 * j] = __float2bfloat16_rn(v[j]);
    if (threadIdx.x == 0) TC_TRACE_POINT(8);
}

int encode_weight_map(CUtensorMap* map, const void* weights, int64_t rows, int64_t hidden) {
    tc::EncodeTiled encode = nullptr;
    int status = tc::encode_entry(&encode);
    if (status != TC_OK) return status;
    cuuint64_t dims[2] = {cuuint64_t(hidden), cuuint64_t(rows)};
    cuuint64_t strides[1] = {cuuint64_t(hidden) * 2};
    cuuint32_t box[2] = {kTileK, kRows};
    cuuint32_t element_strides[2] = {1, 1};
    CUresult result = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(weights), dims, strides, box,
                             element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) return tc::fail(TC_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(result));
    return TC_OK;
}

}  // namespace

extern "C" {

#ifdef TC_TRACE
// Trace builds only: copies the 256 x 16 table of time stamps to `host` (synchronises the device).
int tc_debug_project_trace(void* host) {
    return cudaMemcpyFromSymbol(host, g_project_trace, sizeof(g_project_trace)) == cudaSuccess ? 0 : 1;
}
#endif

int tc_qkv_rope_forward_out(int device, void* stream, const void* x, const void* w_qkv, const void* q_norm_weight,
                            const void* k_norm_weight, const float* rope_cos, const float* rope_sin,
                            int64_t rope_positions, const int32_t* positions, void* q_out, void* knew_out,
                            void* vnew_out, int64_t tokens, int64_t hidden, int64_t q_heads, int64_t kv_heads,
                            double rms_eps) {
    return tc_qkv_rope_forward_out_flags(device, stream, x, w_qkv, q_norm_weight, k_norm_weight, rope_cos, rope_sin,
                                         rope_positions, positions, q_out, knew_out, vnew_out, tokens, hidden, q_heads,
                                         kv_heads, rms_eps, 0);
}

int tc_qkv_rope_forward_out_flags(int device, void* stream, const void* x, const void* w_qkv, const void* q_norm_weight,
                                  const void* k_norm_weight, const float* rope_cos, const float* rope_sin,
                                  int64_t rope_positions, const int32_t* positions, void* q_out, void* knew_out,
                                  void* vnew_out, int64_t tokens, int64_t hidden, int64_t q_heads, int64_t kv_heads,
                                  double rms_eps, int flags) {
    tc::DeviceInfo info;
    int status = tc::require_sm100(device, &info);
    if (status != TC_OK) return status;
    TC_REQUIRE(x && w_qkv && q_out && knew_out && vnew_out, "null tensor pointer");
    TC_REQUIRE((flags & ~TC_PROJECT_RELEASE_EARLY) == 0, "unknown projection flag");
    TC_REQUIRE(tokens >= 1 && tokens <= kMaxTokens, "the projection handles 1 to 8 tokens (one per sequence) per call");
    TC_REQUIRE(hidden >= kTileK && hidden <= kMaxHidden && hidden % kTileK == 0, "hidden must be a multiple of 64 up to 16384");
    TC_REQUIRE(q_heads >= 1 && kv_heads >= 1 && q_heads + 2 * kv_heads <= 4096, "head counts out of range");
    TC_REQUIRE((rope_cos == nullptr) == (rope_sin == nullptr), "pass both RoPE tables or neither");
    TC_REQUIRE(!rope_cos || (positions && rope_positions >= 1), "RoPE needs positions and a non-empty table");
    TC_REQUIRE(std::isfinite(rms_eps) && rms_eps >= 0, "rms_eps must be finite and non-negative");
    const void* aligned[] = {x, w_qkv, q_out, knew_out, vnew_out};
    for (const void* pointer : aligned)
        TC_REQUIRE(reinterpret_cast<uintptr_t>(pointer) % 16 == 0, "16-byte aligned x, weights and outputs required");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    tc::DeviceScratch scratch;
    if ((status = tc::device_scratch(device, &scratch)) != TC_OK) return status;

    const int64_t heads = q_heads + 2 * kv_heads;
    CUtensorMap wmap;
    if ((status = encode_weight_map(&wmap, w_qkv, heads * kRows, hidden)) != TC_OK) return status;
    const int tiles = int(hidden / kTileK);
    int64_t splits = info.sms / heads;  // about one CTA per SM
    splits = splits < 1 ? 1 : (splits > kMaxSplits ? kMaxSplits : splits);
    if (splits > tiles) splits = tiles;
    const int k_local = int((tiles + splits - 1) / splits) * kTileK;
    const int shared = shared_bytes(k_local);
    TC_REQUIRE(shared <= info.smem_optin, "hidden size needs more shared memory than the device offers");

    ProjectParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.q_norm = static_cast<const __nv_bfloat16*>(q_norm_weight);
    p.k_norm = static_cast<const __nv_bfloat16*>(k_norm_weight);
    p.rope_cos = rope_cos;
    p.rope_sin = rope_sin;
    p.positions = positions;
    p.q_out = static_cast<__nv_bfloat16*>(q_out);
    p.k_out = static_cast<__nv_bfloat16*>(knew_out);
    p.v_out = static_cast<__nv_bfloat16*>(vnew_out);
    p.status = scratch.status;
    p.tokens = int(tokens);
    p.hidden = int(hidden);
    p.q_heads = int(q_heads);
    p.kv_heads = int(kv_heads);
    p.splits = int(splits);
    p.rope_positions = int(rope_positions);
    p.eps = float(rms_eps);
    p.release_early = (flags & TC_PROJECT_RELEASE_EARLY) != 0;

    static thread_local int configured_device = -1, configured_shared = 0;
    if (configured_device != device || configured_shared < shared) {
        TC_CUDA(cudaFuncSetAttribute(qkv_rope_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared));
        configured_device = device;
        configured_shared = shared;
    }
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(unsigned(splits), unsigned(heads), 1);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = size_t(shared);
    config.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attributes[2]{};
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = unsigned(splits);
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = 2;
    TC_CUDA(cudaLaunchKernelEx(&config, qkv_rope_kernel, wmap, p));
    return TC_OK;
}

}  // extern "C"
