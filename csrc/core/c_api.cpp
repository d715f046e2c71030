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

// ---- GPU entry points ---------------------------------------------------------------------------------------
// The host core does not link the CUDA runtime. The first GPU call binds the kernel library
// (libnangila_kernels.so, which sits next to this module; NANGILA_KERNELS_LIB overrides the path) with
// dlopen and resolves the few launchers it needs. Counterparts: nangila-hook/src/ffi.rs:526-840.
#include <dlfcn.h>

#include <mutex>
#include <string>

namespace {

struct GpuLib {
  using Stream = void*;
  int64_t (*payload_bytes)(int64_t) = nullptr;
  int (*encode)(const void*, int32_t, const float*, const float*, float*, float, float, int64_t, uint8_t*, Stream) = nullptr;
  int (*decode)(const uint8_t*, int64_t, int32_t, const float*, const float*, float, float, int64_t, float*, Stream) = nullptr;
  int (*crc)(const void*, int64_t, uint32_t*, Stream) = nullptr;
  int64_t (*crc_max)(void) = nullptr;
  int (*to_host)(void*, const void*, int64_t, Stream) = nullptr;
  int (*sync)(Stream) = nullptr;
  bool ok = false;
};

const GpuLib& gpu_lib() {
  static GpuLib lib;
  static std::once_flag once;
  std::call_once(once, [] {
    std::string path;
    if (const char* env = std::getenv("NANGILA_KERNELS_LIB")) path = env;
    if (path.empty()) {
      Dl_info info;
      if (dladdr(reinterpret_cast<void*>(&nangila_free), &info) && info.dli_fname) {
        path = info.dli_fname;
        const size_t slash = path.find_last_of('/');
        path = (slash == std::string::npos ? std::string(".") : path.substr(0, slash)) + "/libnangila_kernels.so";
      }
    }
    void* h = path.empty() ? nullptr : dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
    auto sym = [&](const char* name) { return dlsym(h, name); };
    lib.payload_bytes = reinterpret_cast<decltype(lib.payload_bytes)>(sym("nangila_packet_payload_bytes"));
    lib.encode = reinterpret_cast<decltype(lib.encode)>(sym("nangila_packet_encode"));
    lib.decode = reinterpret_cast<decltype(lib.decode)>(sym("nangila_packet_decode"));
    lib.crc = reinterpret_cast<decltype(lib.crc)>(sym("nangila_crc32_noalloc"));
    lib.crc_max = reinterpret_cast<decltype(lib.crc_max)>(sym("nangila_crc32_noalloc_max_bytes"));
    lib.to_host = reinterpret_cast<decltype(lib.to_host)>(sym("nangila_copy_to_host"));
    lib.sync = reinterpret_cast<decltype(lib.sync)>(sym("nangila_stream_sync"));
    lib.ok = lib.payload_bytes && lib.encode && lib.decode && lib.crc && lib.crc_max && lib.to_host && lib.sync;
  });
  return lib;
}

}  // namespace

NANGILA_EXPORT size_t nangila_gpu_payload_size(size_t count) {
  return 20 + 4 * ((count + 63) / 64) + (count + 1) / 2;
}

NANGILA_EXPORT int32_t nangila_compress_gpu(NangilaHandle h, const float* gradient, const float* g_current,
                                            const float* g_previous, size_t count, uint32_t layer, uint8_t* out_payload,
                                            size_t* out_size, uint8_t* out_header_cpu, void* stream, uint32_t* scratch,
                                            int32_t sync_mode) {
  (void)sync_mode;  // the checksum must reach the host header, so this call always ends with a stream synchronisation
  if (!h || !gradient || !g_current || !g_previous || !out_payload || !out_size || !out_header_cpu || !scratch)
    return NANGILA_INVALID_POINTER;
  const GpuLib& lib = gpu_lib();
  if (!lib.ok || count == 0) return NANGILA_COMPRESSION_ERROR;
  const int64_t payload = lib.payload_bytes(int64_t(count));
  if (payload > lib.crc_max()) return NANGILA_COMPRESSION_ERROR;  // checksum table is a fixed-size device array
  NangilaHook* hook = as_hook(h);
  // kappa < 0: the kernels derive the least-squares gain from the history themselves
  if (lib.encode(gradient, NANGILA_DTYPE_FLOAT32, g_current, g_previous, nullptr, hook->momentum(), -1.0f, int64_t(count),
                 out_payload, stream) != 0)
    return NANGILA_COMPRESSION_ERROR;
  if (lib.crc(out_payload, payload, scratch, stream) != 0) return NANGILA_COMPRESSION_ERROR;
  uint32_t crc = 0;
  if (lib.to_host(&crc, scratch, 4, stream) != 0) return NANGILA_COMPRESSION_ERROR;
  PacketHeader hd = PacketHeader::new_driver(uint32_t(hook->current_step()), layer);
  hd.predictor_hash = hook->predictor_hash();
  hd.crc32 = crc;
  const auto bytes = hd.to_bytes();
  std::memcpy(out_header_cpu, bytes.data(), PacketHeader::SIZE);
  *out_size = PacketHeader::SIZE + size_t(payload);
  return NANGILA_SUCCESS;
}

NANGILA_EXPORT int32_t nangila_decompress_gpu(NangilaHandle h, const uint8_t* compressed, size_t compressed_size,
                                              const float* g_current, const float* g_previous, uint32_t layer,
                                              float* recvbuff, size_t count, void* stream, uint32_t* scratch,
                                              int32_t sync_mode) {
  if (!h || !compressed || !recvbuff || !scratch) return NANGILA_INVALID_POINTER;
  const GpuLib& lib = gpu_lib();
  if (!lib.ok || count == 0 || compressed_size < PacketHeader::SIZE + 20) return NANGILA_DECOMPRESSION_ERROR;
  // header and the fixed words of the payload come to the host first: nothing is launched on a bad packet
  uint8_t head[PacketHeader::SIZE + 12];
  if (lib.to_host(head, compressed, int64_t(sizeof head), stream) != 0) return NANGILA_DECOMPRESSION_ERROR;
  auto hd = PacketHeader::from_bytes(head, PacketHeader::SIZE);
  if (!hd || !hd->is_valid() || hd->layer_id != layer || !hd->is_driver()) return NANGILA_DECOMPRESSION_ERROR;
  float neg_block;
  std::memcpy(&neg_block, head + PacketHeader::SIZE, 4);
  const uint32_t numel = detail::get_le<uint32_t>(head + PacketHeader::SIZE + 4);
  const uint32_t ndim = detail::get_le<uint32_t>(head + PacketHeader::SIZE + 8);
  if (neg_block != -64.0f || numel != count || ndim > 8) return NANGILA_DECOMPRESSION_ERROR;
  const uint8_t* payload = compressed + PacketHeader::SIZE;
  const int64_t payload_bytes = int64_t(compressed_size - PacketHeader::SIZE);
  if (sync_mode != 0) {  // ASYNC (0) skips the checksum, as it skips every other check
    if (payload_bytes > lib.crc_max()) return NANGILA_DECOMPRESSION_ERROR;
    uint32_t crc = 0;
    if (lib.crc(payload, payload_bytes, scratch, stream) != 0 || lib.to_host(&crc, scratch, 4, stream) != 0 || crc != hd->crc32)
      return NANGILA_DECOMPRESSION_ERROR;
  }
  const bool no_pred = (hd->flags & flags::NO_PREDICTION) != 0 || !g_current || !g_previous;
  if (lib.decode(payload, payload_bytes, int32_t(ndim), no_pred ? nullptr : g_current, no_pred ? nullptr : g_previous,
                 as_hook(h)->momentum(), no_pred ? 0.0f : -1.0f, int64_t(count), recvbuff, stream) != 0)
    return NANGILA_DECOMPRESSION_ERROR;
  if (sync_mode == 1 && lib.sync(stream) != 0) return NANGILA_DECOMPRESSION_ERROR;  // ALWAYS: surface launch errors here
  return NANGILA_SUCCESS;
}
