// Compile-time schedule of the causal GQA prefill kernel. The two LSE offsets are the planner's
// answer for the "prefill" handoff and are rewritten by tilecadence_b200.operator.emit; they are
// byte offsets from the start of the CTA's shared-memory arena and must fall inside the released
// terminal K stage [PREFILL_TERMINAL_K_OFFSET_BYTES, +PREFILL_TERMINAL_K_BYTES). The PREFILL_TMEM_*
// values are the planner's tensor-memory map (first column of each tile inside the CTA's
// PREFILL_TMEM_ALLOCATION_COLUMNS allocation), rewritten by the same emitter: score buffers of the
// two heads (equal when the heads share one buffer in alternation), BF16 probability tiles, FP32
// output accumulators.
#pragma once
#define MODEL_FAMILY_CODE 7901
#define PREFILL_BLOCK_M 128
#define PREFILL_BLOCK_N 128
#define PREFILL_GROUP_HEADS 2
#define PREFILL_KV_STAGES 2
#define PREFILL_TERMINAL_K_OFFSET_BYTES 65536
#define PREFILL_TERMINAL_K_BYTES 32768
#define PREFILL_LSE_HEAD0_OFFSET_BYTES 65536
#define PREFILL_LSE_HEAD1_OFFSET_BYTES 66048
#define PREFILL_TMEM_ALLOCATION_COLUMNS 512
#define PREFILL_TMEM_S_HEAD0_COLUMN 0
#define PREFILL_TMEM_S_HEAD1_COLUMN 0
#define PREFILL_TMEM_P_HEAD0_COLUMN 128
#define PREFILL_TMEM_P_HEAD1_COLUMN 192
#define PREFILL_TMEM_O_HEAD0_COLUMN 256
#define PREFILL_TMEM_O_HEAD1_COLUMN 384
