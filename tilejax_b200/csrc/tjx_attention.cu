// Placeholder until the attention kernel lands: the symbol exists so the library matches its header.
#include "tjx_host.cuh"

#include "../../include/tilejax_b200.h"

extern "C" int tjx_causal_attention_bf16(const void*, const void*, const void*, void*, int, int, int, int, int, int,
                                         const int32_t*, const int32_t*, int, int, tjx_stream_t) {
  return tjx::fail(TJX_E_ARG, "tjx_causal_attention_bf16 is not built in this revision");
}
