// Library-level entry points: ABI version, error strings, per-thread CUDA error slot.
#include <stdlib.h>

#include "common.cuh"

namespace uv {
static thread_local int g_last_cuda_error = 0;
void set_last_cuda_error(int e) { g_last_cuda_error = e; }
bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("UVDECODE_PDL");
    return v && v[0] == '1';  // opt-in: measured neutral-to-slightly-slower inside CUDA graphs on B200
  }();
  return on;
}
}  // namespace uv

extern "C" int uv_abi_version(void) { return UV_ABI_VERSION; }

extern "C" int uv_last_cuda_error(void) { return uv::g_last_cuda_error; }

extern "C" const char* uv_error_string(int code) {
  switch (code) {
    case UV_OK: return "ok";
    case UV_ERR_ARG: return "invalid argument (null pointer, negative size or inconsistent options)";
    case UV_ERR_DTYPE: return "dtype not supported by this entry point";
    case UV_ERR_SHAPE: return "shape outside the compiled set (head_dim, group size or vocabulary)";
    case UV_ERR_ALIGN: return "pointer or stride alignment requirement not met";
    case UV_ERR_WORKSPACE: return "workspace missing or too small";
    case UV_ERR_CUDA: return "CUDA runtime error (see uv_last_cuda_error)";
    case UV_ERR_STATIC_LIMIT:
      return "problem exceeds the built-in scratch of uv_decode_attn_static (4 MiB of split partials, 4096 cache rows)";
    default: return "unknown error code";
  }
}
