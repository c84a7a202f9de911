// Compile-time schedule of the split-KV decode kernel. The two *_OFFSET_BYTES values are the
// planner's answer for the "decode" handoff and are rewritten by tilecadence_b200.operator.emit;
// they are byte offsets inside the released terminal V stage (stage 0 of the K/V ring, V first).
#pragma once
#define V10_FAMILY_CODE 7901
#define AB_DECODE_WARPS 4
// Consumer groups of AB_DECODE_WARPS warps that take the tiles in turn. One group keeps 200 registers per
// thread; two groups (288 threads, 112 registers, spills) were slower at every cache length measured.
#ifndef AB_DECODE_WARP_GROUPS
#define AB_DECODE_WARP_GROUPS 1
#endif
#define AB_DECODE_BLOCK_N 64
#ifndef AB_DECODE_STAGES
#define AB_DECODE_STAGES 3
#endif
#define AB_DECODE_STAGE_BYTES 32768
#define AB_DECODE_TERMINAL_V_BYTES 16384
#ifndef AB_DECODE_CTAS_PER_SM
#define AB_DECODE_CTAS_PER_SM 2
#endif
#define AB_DECODE_O_OFFSET_BYTES 0
#define AB_DECODE_LSE_OFFSET_BYTES 2048
