// Host-side launch functions, one set per element type; each lives in its own
// translation unit (inst_f32.cu, inst_bf16.cu, inst_f16.cu, inst_c64.cu) so that the
// library builds in parallel.
#pragma once

#include <cuda_runtime.h>

#include "../../include/ascan_b200.h"

namespace ascan {

struct StreamParams;
struct ShardParams;      // time sharding of the look-back plan (lookback.cuh); null = not sharded

// variant: 0 = plain kinds; 1 = gates are logits, sigmoid fused (real dtypes);
//          2 = complex gates with real tokens (complex64 only)
enum : int { VARIANT_PLAIN = 0, VARIANT_SIGMOID = 1, VARIANT_REAL_TOKENS = 2 };

int launch_f32(int variant, int kind, bool reverse, const StreamParams &p, const ascan_plan &pl, cudaStream_t st,
               const ShardParams *sp = nullptr);
int launch_bf16(int variant, int kind, bool reverse, const StreamParams &p, const ascan_plan &pl, cudaStream_t st,
               const ShardParams *sp = nullptr);
int launch_f16(int variant, int kind, bool reverse, const StreamParams &p, const ascan_plan &pl, cudaStream_t st,
               const ShardParams *sp = nullptr);
int launch_c64(int variant, int kind, bool reverse, const StreamParams &p, const ascan_plan &pl, cudaStream_t st,
               const ShardParams *sp = nullptr);

}  // namespace ascan
