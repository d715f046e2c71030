// C ABI over the C++ hook state machine (see nangila_ffi.h).
#include "nangila_ffi.h"

#include <cstring>

#include "dtype.hpp"
#include "hook.hpp"

#define NANGILA_EXPORT extern "C" __attribute__((visibility("default")))

using namespace nangila;

namespace {
NangilaHook* as_hook(NangilaHandle h) { return static_cast<NangilaHook*>(h); }
}  // namespace

NANGILA_EXPORT NangilaHandle nangila_init(const char* mask_path) {
  if (mask_path == nullptr) return nullptr;
  try {
    return new NangilaHook(NangilaHook::from_mask_file(mask_path));
  } catch (...) {
    return nullptr;
  }
}
NANGILA_EXPORT NangilaHandle nangila_init_all_drivers(uint32_t num_layers) {
  try {
    return new NangilaHook(NangilaHook::all_drivers(num_layers));
  } catch (...) {
    return nullptr;
  }
}
NANGILA_EXPORT NangilaHandle nangila_init_all_drivers_ex(uint32_t num_layers, uint64_t warmup, uint64_t shadow) {
  try {
    NangilaConfig c;
    c.warmup_steps = size_t(warmup);
    c.shadow_run_steps = size_t(shadow);
    return new NangilaHook(NangilaHook::all_drivers(num_layers, c));
  } catch (...) {
    return nullptr;
  }
}
NANGILA_EXPORT void nangila_free(NangilaHandle h) { delete as_hook(h); }
NANGILA_EXPORT void nangila_set_gpu_mode(NangilaHandle h, int32_t enabled) {
  if (h) as_hook(h)->set_gpu_mode(enabled != 0);
}

NANGILA_EXPORT int32_t nangila_compress_ex(NangilaHandle h, const uint8_t* send, size_t count, int32_t dtype, uint32_t layer,
                                           uint8_t* out, size_t* out_size) {
  if (!h || !send || !out || !out_size) return NANGILA_INVALID_POINTER;
  DataType dt;
  if (!data_type_from_i32(dtype, &dt)) return NANGILA_COMPRESSION_ERROR;
  try {
    std::vector<uint8_t> pkt = as_hook(h)->on_send(layer, tensor_from_bytes(send, count, dt));
    std::memcpy(out, pkt.data(), pkt.size());
    *out_size = pkt.size();
    return NANGILA_SUCCESS;
  } catch (...) {
    return NANGILA_COMPRESSION_ERROR;
  }
}
NANGILA_EXPORT int32_t nangila_compress(NangilaHandle h, const float* send, size_t count, uint32_t layer, uint8_t* out,
                                        size_t* out_size) {
  return nangila_compress_ex(h, reinterpret_cast<const uint8_t*>(send), count, NANGILA_DTYPE_FLOAT32, layer, out, out_size);
}
NANGILA_EXPORT int32_t nangila_decompress_ex(NangilaHandle h, const uint8_t* compressed, size_t size, uint32_t layer,
                                             uint8_t* recv, size_t count, int32_t dtype) {
  if (!h || !compressed || !recv) return NANGILA_INVALID_POINTER;
  DataType dt;
  if (!data_type_from_i32(dtype, &dt)) return NANGILA_DECOMPRESSION_ERROR;
  try {
    Tensor t = as_hook(h)->on_receive(layer, compressed, size);
    if (t.numel() != count) return NANGILA_DECOMPRESSION_ERROR;
    tensor_to_bytes(t, dt, recv);
    return NANGILA_SUCCESS;
  } catch (...) {
    return NANGILA_DECOMPRESSION_ERROR;
  }
}
NANGILA_EXPORT int32_t nangila_decompress(NangilaHandle h, const uint8_t* compressed, size_t size, uint32_t layer,
                                          float* recv, size_t count) {
  return nangila_decompress_ex(h, compressed, size, layer, reinterpret_cast<uint8_t*>(recv), count, NANGILA_DTYPE_FLOAT32);
}
NANGILA_EXPORT int32_t nangila_on_complete(NangilaHandle h, const float* g, size_t count, uint32_t layer) {
  if (!h || !g) return NANGILA_INVALID_POINTER;
  as_hook(h)->on_complete(layer, Tensor::from_slice(g, count));
  return NANGILA_SUCCESS;
}
NANGILA_EXPORT int32_t nangila_step(NangilaHandle h) {
  if (!h) return NANGILA_INVALID_POINTER;
  as_hook(h)->step();
  return NANGILA_SUCCESS;
}
NANGILA_EXPORT int32_t nangila_is_enabled(NangilaHandle h) { return h && as_hook(h)->is_compression_enabled() ? 1 : 0; }
NANGILA_EXPORT uint64_t nangila_current_step(NangilaHandle h) { return h ? uint64_t(as_hook(h)->current_step()) : 0; }
NANGILA_EXPORT uint64_t nangila_predictor_hash(NangilaHandle h) { return h ? as_hook(h)->predictor_hash() : 0; }
NANGILA_EXPORT size_t nangila_max_compressed_size(size_t count) { return 16 + 12 + 4 * count + 32; }

NANGILA_EXPORT void nangila_enable_safe_mode(NangilaHandle h, float divergence_threshold, size_t check_interval,
                                             uint32_t max_consecutive_failures, size_t recovery_cooldown) {
  if (!h) return;
  SafeModeConfig c;
  c.divergence_threshold = divergence_threshold;
  c.check_interval = check_interval;
  c.max_consecutive_failures = max_consecutive_failures;
  c.recovery_cooldown = recovery_cooldown;
  as_hook(h)->enable_safe_mode(c);
}
NANGILA_EXPORT int32_t nangila_report_val_loss(NangilaHandle h, float loss) {
  if (!h) return 3;
  return int32_t(as_hook(h)->report_validation_loss(loss));
}
