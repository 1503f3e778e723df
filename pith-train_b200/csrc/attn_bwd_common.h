// Shared between the two attention-backward translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pith_b200.h"

namespace pith {

enum BwdMode : int { kDkDv = 0, kDq = 1 };

struct BwdParams {
  const float* lse;
  const float* delta;
  float* dq_acc;
  float* dk_acc;
  float* dv_acc;
  uint32_t* status;
  int B, Sq, Sk, Hq, Hkv;
  int causal, causal_off;
  int hpc;            // head_dim-128 dK/dV pass: query heads per CTA (set by its launcher)
  int dq_store_bf16;  // dq_acc points at a bf16 [B][Sq][Hq][D] OUTPUT that the dQ pass stores (dqs in bf16 elements)
  float scale_log2, scale;
  int64_t dqs[3], dks[3], dvs[3];
  int64_t ls[2], dls[2];
};

// Head dimension 128 (GQA / MHA) with 128-wide streamed tiles (attn_bwd128.cu).
int launch_bwd_d128(const pith_attn_bwd_args* a, const BwdParams& p, int mode, cudaStream_t st);

}  // namespace pith
