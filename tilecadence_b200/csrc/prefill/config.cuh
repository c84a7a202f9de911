// Compile-time schedule of the causal GQA prefill kernel. The two LSE offsets are the planner's
// answer for the "prefill" handoff and are rewritten by tilecadence_b200.operator.emit; they are
// byte offsets from the start of the CTA's shared-memory arena and must fall inside the released
// terminal K stage [PREFILL_TERMINAL_K_OFFSET_BYTES, +PREFILL_TERMINAL_K_BYTES).
#pragma once
#define MODEL_FAMILY_CODE 7901
#define PREFILL_BLOCK_M 128
#define PREFILL_BLOCK_N 128
#define PREFILL_GROUP_HEADS 2
#define PREFILL_KV_STAGES 2
#ifndef PREFILL_MAX3
#define PREFILL_MAX3 1
#endif
#ifndef PREFILL_PACKED_MATH
#define PREFILL_PACKED_MATH 1
#endif
#ifndef PREFILL_SETMAXNREG
#define PREFILL_SETMAXNREG 1
#endif
#ifndef PREFILL_TURN_NAMED
#define PREFILL_TURN_NAMED 1
#endif
#ifndef PREFILL_TURN_CHUNK
#define PREFILL_TURN_CHUNK 3
#endif
#ifndef PREFILL_PINGPONG
#define PREFILL_PINGPONG 1
#endif
#ifndef PREFILL_SPLIT_P
#define PREFILL_SPLIT_P 1
#endif
#ifndef PREFILL_EARLY_P
#define PREFILL_EARLY_P 1
#endif
#ifndef PREFILL_WARP_ARRIVE
#define PREFILL_WARP_ARRIVE 0
#endif
#ifndef PREFILL_SHADOW_CHUNKS
#define PREFILL_SHADOW_CHUNKS 0
#endif
#ifndef PREFILL_EXP_FMA_PAIRS_PER_8
#define PREFILL_EXP_FMA_PAIRS_PER_8 0
#endif
#define PREFILL_TERMINAL_K_OFFSET_BYTES 65536
#define PREFILL_TERMINAL_K_BYTES 32768
#define PREFILL_LSE_HEAD0_OFFSET_BYTES 65536
#define PREFILL_LSE_HEAD1_OFFSET_BYTES 66048
