// placeholder until the backward kernel lands
#include "../../include/pith_b200.h"
#include "host_common.h"
extern "C" int pith_attn_bwd(const pith_attn_bwd_args* a, void* stream) {
  (void)a; (void)stream;
  return pith::fail(pith::kErrUnsupported, "pith_attn_bwd is not built yet");
}
