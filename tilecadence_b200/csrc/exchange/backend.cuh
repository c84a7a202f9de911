// Primitive library for the generated two-tile attention kernel (one CTA = 64 queries x 64 keys x
// D128 for one (batch, head); 4 warps, warp w owns query rows 16w..16w+15).
//
// Counterpart of tilecadence/cuda/exchange/backend.cuh (issue_g2s :58-67, load_operand_ready :82-101,
// load_v_ready :103-122, store/load_checkpoint :135-166, qk :195-202, stats_first/next :226-275,
// pv :292-297, rescale :299-307, normalize_store_coalesced128 :309-407, store_lse :409-420) for
// sm_100a, without CuTe: global-to-shared copies are TMA tile copies (128-byte swizzle) that each arm
// their own transaction mbarrier; "ready" loads observe every barrier armed since the last wait and
// meet at a CTA barrier; operands live in registers as mma.sync.m16n8k16 fragments read with ldmatrix
// from the swizzled slabs. The emitted kernel is a straight line of calls in the planner's order.
#pragma once
#include "tc_ptx.cuh"

#ifndef TC_EXCHANGE_OUTPUT_STREAMING_STORE
#define TC_EXCHANGE_OUTPUT_STREAMING_STORE 0
#endif

namespace tc_exchange {

constexpr float kScale = 0.08838834764831845f;           // 128^-0.5
constexpr float kScaleLog2 = kScale * 1.4426950408889634f;
constexpr int kMaxCopies = 16;

struct Context {
    unsigned char* arena;   // 1024-byte aligned dynamic shared memory, 8 slabs of 4 KiB
    uint64_t* barriers;     // one single-use mbarrier per copy_g2s, in issue order
    int32_t* status;        // device status word for expired waits
    int batch, head;
    int warp, group, quad;  // warp index, lane / 4, lane % 4
};

template <class Element> struct OperandQ { uint32_t a[8][4]; };     // 16 rows x D128: 8 k-steps
template <class Element> struct OperandK { uint32_t b[8][4][2]; };  // 32 keys x D128: [k-step][n-tile]
template <class Element> struct OperandV { uint32_t b[2][8][2]; };  // 32 keys x 64 d: [k-step][n-tile]
template <class Element> struct Probabilities { uint32_t a[2][4]; };  // 16 rows x 32 keys
struct Scores { float c[4][4]; };                                   // 16 rows x 32 keys, fp32
struct Accumulator { float c[8][4]; };                              // 16 rows x 64 d, fp32
struct RowPair { float v[2]; };                                     // rows group and group + 8

__device__ __forceinline__ uint32_t swizzled(uint32_t row, uint32_t chunk16, uint32_t half_bytes) {
    // 16-byte chunk `chunk16` of row `row` in a tile stored as 64-column halves with 128-byte rows.
    return (chunk16 >> 3) * half_bytes + row * 128 + (((chunk16 & 7) ^ (row & 7)) << 4);
}

template <class Element> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) { return tc::pack_f16x2(lo, hi); }
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) { return tc::pack_bf16x2(lo, hi); }

template <class Element>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    tc::mma_bf16_16816(d, a[0], a[1], a[2], a[3], b[0], b[1]);
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ Context make_context(unsigned char* arena, uint64_t* barriers, int32_t* status) {
    Context ctx;
    ctx.arena = arena;
    ctx.barriers = barriers;
    ctx.status = status;
    ctx.batch = blockIdx.y;
    ctx.head = blockIdx.z;
    ctx.warp = threadIdx.x >> 5;
    ctx.group = (threadIdx.x & 31) >> 2;
    ctx.quad = threadIdx.x & 3;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kMaxCopies; ++i) tc::mbar_init(&barriers[i], 1);
        tc::mbar_fence_init();
    }
    __syncthreads();
    return ctx;
}

// copy_g2s: ROWS x COLS elements starting at (row0, col0) of this (batch, head) into a slab span.
// One thread arms barrier `index` with the byte count and issues one TMA copy per 64-column half.
template <class Element, int ROWS, int COLS, int INDEX>
__device__ __forceinline__ void issue_g2s(const Context& ctx, const CUtensorMap* map, int row0, int col0,
                                          unsigned char* destination) {
    static_assert(INDEX < kMaxCopies && (COLS == 64 || COLS == 128), "copy geometry");
    if (threadIdx.x == 0) {
        const uint64_t policy = tc::policy_evict_first();
        tc::mbar_arrive_expect_tx(&ctx.barriers[INDEX], ROWS * COLS * 2);
#pragma unroll
        for (int half = 0; half < COLS / 64; ++half)
            tc::tma_load_4d(destination + half * (ROWS * 128), map, &ctx.barriers[INDEX], col0 + half * 64, ctx.head,
                            row0, ctx.batch, policy);
    }
}

// Wait before a load whose copy is newer than the ready cutoff: observe every barrier armed since the
// previous wait, then meet at a CTA barrier (which also retires all earlier distributed shared reads).
template <int FIRST, int LAST>
__device__ __forceinline__ void acquire_copies(const Context& ctx) {
    bool ok = true;
#pragma unroll
    for (int i = FIRST; i < LAST; ++i) ok = tc::mbar_wait(&ctx.barriers[i], 0) && ok;
    if (!ok) atomicCAS(ctx.status, 0, 31);
    __syncthreads();
}

// A shared write is about to land on slabs that other threads may still be reading.
__device__ __forceinline__ void release_shared_reads() { __syncthreads(); }

template <class Element>
__device__ __forceinline__ OperandQ<Element> load_q_ready(const Context& ctx, const unsigned char* slab) {
    OperandQ<Element> q;
    const uint32_t base = tc::smem_u32(slab);
    const int lane = threadIdx.x & 31, mat = lane >> 3;
    const uint32_t row = uint32_t(ctx.warp * 16 + (mat & 1) * 8 + (lane & 7));
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
        tc::ldmatrix_x4(base + swizzled(row, uint32_t(ks * 2 + (mat >> 1)), 64 * 128), q.a[ks][0], q.a[ks][1], q.a[ks][2],
                        q.a[ks][3]);
    return q;
}

template <class Element>
__device__ __forceinline__ OperandK<Element> load_k_ready(const Context& ctx, const unsigned char* slab) {
    OperandK<Element> k;
    const uint32_t base = tc::smem_u32(slab);
    const int lane = threadIdx.x & 31, mat = lane >> 3;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
#pragma unroll
        for (int pair = 0; pair < 2; ++pair) {
            // matrices: (keys n0.., d lo) (keys n0.., d hi) (keys n0+8.., d lo) (keys n0+8.., d hi)
            const uint32_t row = uint32_t(pair * 16 + (mat >> 1) * 8 + (lane & 7));
            tc::ldmatrix_x4(base + swizzled(row, uint32_t(ks * 2 + (mat & 1)), 32 * 128), k.b[ks][2 * pair][0],
                            k.b[ks][2 * pair][1], k.b[ks][2 * pair + 1][0], k.b[ks][2 * pair + 1][1]);
        }
    return k;
}

template <class Element>
__device__ __forceinline__ OperandV<Element> load_v_ready(const Context& ctx, const unsigned char* slab) {
    OperandV<Element> v;
    const uint32_t base = tc::smem_u32(slab);
    const int lane = threadIdx.x & 31, mat = lane >> 3;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk)
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            // matrices: (keys 0-7, d n0) (keys 8-15, d n0) (keys 0-7, d n0+1) (keys 8-15, d n0+1), transposed
            const uint32_t row = uint32_t(kk * 16 + (mat & 1) * 8 + (lane & 7));
            tc::ldmatrix_x4_trans(base + swizzled(row, uint32_t(np * 2 + (mat >> 1)), 32 * 128), v.b[kk][2 * np][0],
                                  v.b[kk][2 * np][1], v.b[kk][2 * np + 1][0], v.b[kk][2 * np + 1][1]);
        }
    return v;
}

// Checkpoint: P as a row-major 64 x 32 tile of Elements (64-byte rows) in one slab, then a CTA barrier.
template <class Element>
__device__ __forceinline__ void store_checkpoint(const Probabilities<Element>& p, Element* slab, const Context& ctx) {
    uint32_t* words = reinterpret_cast<uint32_t*>(slab);
    const int row = ctx.warp * 16 + ctx.group;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
        words[row * 16 + kk * 8 + ctx.quad] = p.a[kk][0];
        words[(row + 8) * 16 + kk * 8 + ctx.quad] = p.a[kk][1];
        words[row * 16 + kk * 8 + 4 + ctx.quad] = p.a[kk][2];
        words[(row + 8) * 16 + kk * 8 + 4 + ctx.quad] = p.a[kk][3];
    }
    __syncthreads();
}

template <class Element>
__device__ __forceinline__ Probabilities<Element> load_checkpoint(const Element* slab, const Context& ctx) {
    Probabilities<Element> p;
    const uint32_t* words = reinterpret_cast<const uint32_t*>(slab);
    const int row = ctx.warp * 16 + ctx.group;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
        p.a[kk][0] = words[row * 16 + kk * 8 + ctx.quad];
        p.a[kk][1] = words[(row + 8) * 16 + kk * 8 + ctx.quad];
        p.a[kk][2] = words[row * 16 + kk * 8 + 4 + ctx.quad];
        p.a[kk][3] = words[(row + 8) * 16 + kk * 8 + 4 + ctx.quad];
    }
    return p;
}

template <class Element>
__device__ __forceinline__ Scores qk(const OperandQ<Element>& q, const OperandK<Element>& k) {
    Scores s;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s.c[nt][0] = s.c[nt][1] = s.c[nt][2] = s.c[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) mma16816<Element>(s.c[nt], q.a[ks], k.b[ks][nt]);
    return s;
}

template <bool Causal, int Tile>
__device__ __forceinline__ void mask_scores(const Context& ctx, Scores& s) {
    if constexpr (Causal) {
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = ctx.warp * 16 + ctx.group + (i >> 1) * 8;
                const int col = Tile * 32 + nt * 8 + ctx.quad * 2 + (i & 1);
                if (col > row) s.c[nt][i] = -INFINITY;
            }
    }
}

__device__ __forceinline__ float quad_max(float x) {
    x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
    return fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
}
__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x + __shfl_xor_sync(0xffffffffu, x, 2);
}

template <class Element>
__device__ __forceinline__ void exponentiate(const Scores& s, const RowPair& m, RowPair& sum, Probabilities<Element>& p) {
    float e[4][4];
    sum.v[0] = sum.v[1] = 0.f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float reference = m.v[i >> 1] == -INFINITY ? 0.f : m.v[i >> 1];
            e[nt][i] = tc::fast_exp2((s.c[nt][i] - reference) * kScaleLog2);
            sum.v[i >> 1] += e[nt][i];
        }
    sum.v[0] = quad_sum(sum.v[0]);  // full row sums, replicated across the quad
    sum.v[1] = quad_sum(sum.v[1]);
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
        p.a[kk][0] = pack2<Element>(e[2 * kk][0], e[2 * kk][1]);
        p.a[kk][1] = pack2<Element>(e[2 * kk][2], e[2 * kk][3]);
        p.a[kk][2] = pack2<Element>(e[2 * kk + 1][0], e[2 * kk + 1][1]);
        p.a[kk][3] = pack2<Element>(e[2 * kk + 1][2], e[2 * kk + 1][3]);
    }
}

// First key tile: row maximum, probabilities and full row sum.
template <bool Causal, int Tile, class Element>
__device__ __forceinline__ void stats_first(const Context& ctx, Scores s, RowPair& m, RowPair& l, Probabilities<Element>& p) {
    mask_scores<Causal, Tile>(ctx, s);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float x = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) x = fmaxf(x, fmaxf(s.c[nt][2 * r], s.c[nt][2 * r + 1]));
        m.v[r] = quad_max(x);
    }
    exponentiate<Element>(s, m, l, p);
}

// Later key tile: new maximum, rescale factor for what was accumulated so far, updated row sum.
template <bool Causal, int Tile, class Element>
__device__ __forceinline__ void stats_next(const Context& ctx, Scores s, const RowPair& m_before, const RowPair& l_before,
                                           RowPair& m, RowPair& l, RowPair& alpha, Probabilities<Element>& p) {
    mask_scores<Causal, Tile>(ctx, s);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float x = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) x = fmaxf(x, fmaxf(s.c[nt][2 * r], s.c[nt][2 * r + 1]));
        m.v[r] = fmaxf(m_before.v[r], quad_max(x));
        alpha.v[r] = m_before.v[r] == -INFINITY ? 0.f : tc::fast_exp2((m_before.v[r] - m.v[r]) * kScaleLog2);
    }
    RowPair tile_sum;
    exponentiate<Element>(s, m, tile_sum, p);
    l.v[0] = fmaf(l_before.v[0], alpha.v[0], tile_sum.v[0]);
    l.v[1] = fmaf(l_before.v[1], alpha.v[1], tile_sum.v[1]);
}

__device__ __forceinline__ void clear(Accumulator& o) {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) o.c[nt][0] = o.c[nt][1] = o.c[nt][2] = o.c[nt][3] = 0.f;
}

template <class Element>
__device__ __forceinline__ void pv(const Probabilities<Element>& p, const OperandV<Element>& v, Accumulator& o) {
#pragma unroll
    for (int kk = 0; kk < 2; ++kk)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) mma16816<Element>(o.c[nt], p.a[kk], v.b[kk][nt]);
}

__device__ __forceinline__ void rescale(Accumulator& o, const RowPair& alpha) {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        o.c[nt][0] *= alpha.v[0];
        o.c[nt][1] *= alpha.v[0];
        o.c[nt][2] *= alpha.v[1];
        o.c[nt][3] *= alpha.v[1];
    }
}

// Close one 64-wide output stripe: normalise, convert, stage the 64 x 64 tile in the 8 KiB scratch span
// (128-byte rows, chunk-swizzled), one CTA barrier, then 16-byte coalesced stores to O[b, row, h, :].
template <class Element, int Stripe>
__device__ __forceinline__ void normalize_store_coalesced128(const Context& ctx, const Accumulator& o, const RowPair& l,
                                                             Element* o_base, int row_stride, unsigned char* scratch) {
    const float inv0 = l.v[0] > 0.f ? 1.f / l.v[0] : 0.f, inv1 = l.v[1] > 0.f ? 1.f / l.v[1] : 0.f;
    const int row = ctx.warp * 16 + ctx.group;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        // 4-byte word at column nt*8 + quad*2 of rows `row` and `row + 8`
        const uint32_t word = uint32_t(ctx.quad) * 4;
        *reinterpret_cast<uint32_t*>(scratch + row * 128 + ((nt ^ (row & 7)) << 4) + word) =
            pack2<Element>(o.c[nt][0] * inv0, o.c[nt][1] * inv0);
        *reinterpret_cast<uint32_t*>(scratch + (row + 8) * 128 + ((nt ^ ((row + 8) & 7)) << 4) + word) =
            pack2<Element>(o.c[nt][2] * inv1, o.c[nt][3] * inv1);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int index = int(threadIdx.x) + i * 128;  // 512 chunks of 16 bytes
        const int r = index >> 3, chunk = index & 7;
        const uint4 value = *reinterpret_cast<const uint4*>(scratch + r * 128 + ((chunk ^ (r & 7)) << 4));
        uint4* destination = reinterpret_cast<uint4*>(o_base + int64_t(r) * row_stride + Stripe * 64 + chunk * 8);
#if TC_EXCHANGE_OUTPUT_STREAMING_STORE
        __stcs(destination, value);
#else
        *destination = value;
#endif
    }
}

// LSE = m * scale + ln(l), natural log; +inf for a row without any visible key.
__device__ __forceinline__ void store_lse(const Context& ctx, const RowPair& m, const RowPair& l, float* lse_base) {
    if (ctx.quad == 0) {
        const int row = ctx.warp * 16 + ctx.group;
        lse_base[row] = l.v[0] > 0.f ? fmaf(m.v[0], kScale, logf(l.v[0])) : INFINITY;
        lse_base[row + 8] = l.v[1] > 0.f ? fmaf(m.v[1], kScale, logf(l.v[1])) : INFINITY;
    }
}

}  // namespace tc_exchange
