// Generated from planner events, concrete copy bindings and shared byte offsets: do not edit.
// Complete attention for 64 queries x 64 keys, D128, two 64-wide output stripes, one CTA per (batch, head).
#define TC_EXCHANGE_OUTPUT_STREAMING_STORE 0
#include "backend.cuh"
#include "tc_host.cuh"

namespace {
using namespace tc_exchange;
template <class Element, bool Causal>
__global__ void __launch_bounds__(128) solver_attention(const __grid_constant__ CUtensorMap qmap,
    const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, Element* O, float* LSE,
    int H, int32_t* status) {
    static_assert(sizeof(Element) == 2);
    extern __shared__ unsigned char arena_raw[];
    unsigned char* arena = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(arena_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t barriers[kMaxCopies];
    const Context ctx = make_context(arena, barriers, status);
    const int row_stride = H * 128;
    Element* o_base = O + (int64_t(ctx.batch) * 64 * H + ctx.head) * 128;
    float* lse_base = LSE + (int64_t(ctx.batch) * H + ctx.head) * 64;
    unsigned char* s9=arena+0;
    unsigned char* s11=arena+0;
    unsigned char* s14=arena+0;
    unsigned char* s16=arena+16384;
    unsigned char* s19=arena+20480;
    Element* s21=reinterpret_cast<Element*>(arena+4096);
    unsigned char* s23=arena+16384;
    Element* s25=reinterpret_cast<Element*>(arena+0);
    unsigned char* s28=arena+16384;
    unsigned char* s30=arena+16384;
    // EVENT copy_K0#0
    issue_g2s<Element,32,128,0>(ctx,&kmap,0,0,s9);
    // EVENT load_K0#0
    acquire_copies<0,1>(ctx);  // copy newer than the ready cutoff
    auto r8=load_k_ready<Element>(ctx,s9);
    // EVENT copy_K1#0
    release_shared_reads();  // this shared write overlaps slabs with distributed reads outstanding
    issue_g2s<Element,32,128,1>(ctx,&kmap,32,0,s14);
    // EVENT load_K1#0
    acquire_copies<1,2>(ctx);  // copy newer than the ready cutoff
    auto r13=load_k_ready<Element>(ctx,s14);
    // EVENT copy_Q#0
    release_shared_reads();  // this shared write overlaps slabs with distributed reads outstanding
    issue_g2s<Element,64,128,2>(ctx,&qmap,0,0,s11);
    // EVENT load_Q#0
    acquire_copies<2,3>(ctx);  // copy newer than the ready cutoff
    auto r10=load_q_ready<Element>(ctx,s11);
    // EVENT qk_0#0
    auto r7=qk<Element>(r10,r8);
    // EVENT stats_0#0
    RowPair r4;
    RowPair r5;
    Probabilities<Element> r6;
    stats_first<Causal,0,Element>(ctx,r7,r4,r5,r6);
    // EVENT store_P0#0
    release_shared_reads();  // this shared write overlaps slabs with distributed reads outstanding
    store_checkpoint(r6,s25,ctx);
    // EVENT copy_V0_0#0
    issue_g2s<Element,32,64,3>(ctx,&vmap,0,0,s30);
    // EVENT load_V0_0#0
    acquire_copies<3,4>(ctx);  // copy newer than the ready cutoff
    auto r29=load_v_ready<Element>(ctx,s30);
    // EVENT pv_0_0#0
    Accumulator o0;
    clear(o0);  // the stripe's register lifetime begins here
    pv<Element>(r6,r29,o0);
    // EVENT copy_Q#1
    release_shared_reads();  // this shared write overlaps slabs with distributed reads outstanding
    issue_g2s<Element,64,128,4>(ctx,&qmap,0,0,s16);
    // EVENT load_Q#1
    acquire_copies<4,5>(ctx);  // copy newer than the ready cutoff
    auto r15=load_q_ready<Element>(ctx,s16);
    // EVENT qk_1#0
    auto r12=qk<Element>(r15,r13);
    // EVENT stats_1#0
    RowPair r0;
    RowPair r1;
    RowPair r2;
    Probabilities<Element> r3;
    stats_next<Causal,1,Element>(ctx,r12,r4,r5,r0,r1,r2,r3);
    // EVENT store_lse#0
    store_lse(ctx,r0,r1,lse_base);
    // EVENT rescale_1_0#0
    rescale(o0,r2);
    // EVENT copy_V1_0#0
    release_shared_reads();  // this shared write overlaps slabs with distributed reads outstanding
    issue_g2s<Element,32,64,5>(ctx,&vmap,32,0,s28);
    // EVENT load_V1_0#0
    acquire_copies<5,6>(ctx);  // copy newer than the ready cutoff
    auto r27=load_v_ready<Element>(ctx,s28);
    // EVENT pv_1_0#0
    pv<Element>(r3,r27,o0);
    // EVENT close_0#0
    release_shared_reads();  // this shared write overlaps slabs with distributed reads outstanding
    normalize_store_coalesced128<Element,0>(ctx,o0,r1,o_base,row_stride,arena+16384);
    // EVENT store_P1#0
    store_checkpoint(r3,s21,ctx);
    // EVENT copy_V0_1#0
    issue_g2s<Element,32,64,6>(ctx,&vmap,0,64,s23);
    // EVENT copy_V1_1#0
    issue_g2s<Element,32,64,7>(ctx,&vmap,32,64,s19);
    // EVENT load_P0#0
    auto r24=load_checkpoint<Element>(s25,ctx);
    // EVENT load_V0_1#0
    acquire_copies<6,8>(ctx);  // copy newer than the ready cutoff
    auto r22=load_v_ready<Element>(ctx,s23);
    // EVENT pv_0_1#0
    Accumulator o1;
    clear(o1);  // the stripe's register lifetime begins here
    pv<Element>(r24,r22,o1);
    // EVENT rescale_1_1#0
    rescale(o1,r2);
    // EVENT load_P1#0
    auto r20=load_checkpoint<Element>(s21,ctx);
    // EVENT load_V1_1#0
    auto r18=load_v_ready<Element>(ctx,s19);
    // EVENT pv_1_1#0
    pv<Element>(r20,r18,o1);
    // EVENT close_1#0
    release_shared_reads();  // this shared write overlaps slabs with distributed reads outstanding
    normalize_store_coalesced128<Element,1>(ctx,o1,r1,o_base,row_stride,arena+16384);
}

constexpr int kArenaBytes = 32768;
constexpr int kDynamicShared = kArenaBytes + 1024;  // slack for the 1024-byte alignment of the arena

template <class Element, bool Causal>
int launch(const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap, void* out, float* lse,
           int64_t batch, int64_t heads, int32_t* status, cudaStream_t stream) {
    auto kernel = &solver_attention<Element, Causal>;
    TC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynamicShared));
    kernel<<<dim3(1, unsigned(batch), unsigned(heads)), 128, kDynamicShared, stream>>>(
        qmap, kmap, vmap, static_cast<Element*>(out), lse, int(heads), status);
    TC_CUDA(cudaGetLastError());
    return TC_OK;
}

template <class Element, bool Causal>
int describe(int64_t* values) {
    int64_t attributes[8];
    int status = tc::kernel_resources(&solver_attention<Element, Causal>, 128, kDynamicShared, attributes);
    if (status != TC_OK) return status;
    const int64_t row[14] = {64, 32, 128, 64, attributes[0], attributes[1], attributes[2], attributes[3],
                             attributes[4], attributes[5], attributes[6], attributes[7], 0, 0};
    for (int i = 0; i < 14; ++i) values[i] = row[i];
    return TC_OK;
}

}  // namespace

extern "C" {

int tc_exchange_forward_out(int device, void* stream, const void* q, const void* k, const void* v, void* out,
                            float* lse, int64_t batch, int64_t heads, int dtype_fp16, int causal) {
    tc::DeviceInfo info;
    int status = tc::require_sm100(device, &info);
    if (status != TC_OK) return status;
    TC_REQUIRE(q && k && v && out && lse, "null tensor pointer");
    TC_REQUIRE(batch > 0 && batch <= 65535 && heads > 0 && heads <= 65535, "B and H must be positive and fit the CUDA grid");
    const size_t bytes = size_t(batch) * 64 * heads * 128 * 2, lse_bytes = size_t(batch) * heads * 64 * 4;
    for (const void* pointer : {q, k, v, static_cast<const void*>(out)})
        TC_REQUIRE(reinterpret_cast<uintptr_t>(pointer) % 16 == 0, "16-byte aligned Q/K/V/O required");
    for (const void* input : {q, k, v})
        TC_REQUIRE(!tc::ranges_overlap(out, bytes, input, bytes) && !tc::ranges_overlap(lse, lse_bytes, input, bytes),
                   "Outputs may not alias inputs");
    TC_REQUIRE(!tc::ranges_overlap(out, bytes, lse, lse_bytes), "Outputs may not alias each other");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    tc::DeviceScratch scratch;
    if ((status = tc::device_scratch(device, &scratch)) != TC_OK) return status;
    CUtensorMap qmap, kmap, vmap;
    const bool fp16 = dtype_fp16 != 0;
    if ((status = tc::make_rows_map(&qmap, q, fp16, heads, 64, batch, 128, heads * 128, 64 * heads * 128, 64, 2)) != TC_OK) return status;
    if ((status = tc::make_rows_map(&kmap, k, fp16, heads, 64, batch, 128, heads * 128, 64 * heads * 128, 32, 2)) != TC_OK) return status;
    if ((status = tc::make_rows_map(&vmap, v, fp16, heads, 64, batch, 128, heads * 128, 64 * heads * 128, 32, 2)) != TC_OK) return status;
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (fp16)
        return causal ? launch<__half, true>(qmap, kmap, vmap, out, lse, batch, heads, scratch.status, s)
                      : launch<__half, false>(qmap, kmap, vmap, out, lse, batch, heads, scratch.status, s);
    return causal ? launch<__nv_bfloat16, true>(qmap, kmap, vmap, out, lse, batch, heads, scratch.status, s)
                  : launch<__nv_bfloat16, false>(qmap, kmap, vmap, out, lse, batch, heads, scratch.status, s);
}

int tc_exchange_resources(int device, int dtype_fp16, int causal, int64_t values[14]) {
    tc::DeviceInfo info;
    int status = tc::require_sm100(device, &info);
    if (status != TC_OK) return status;
    TC_REQUIRE(values, "null values");
    tc::DeviceGuard guard(device);
    TC_CUDA(guard.status);
    if (dtype_fp16) return causal ? describe<__half, true>(values) : describe<__half, false>(values);
    return causal ? describe<__nv_bfloat16, true>(values) : describe<__nv_bfloat16, false>(values);
}

}  // extern "C"
