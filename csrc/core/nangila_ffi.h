/* C ABI of the host-side core, for embedding the hook state machine in a C or C++ runtime.
 * Function names, argument orders and result codes follow the reference
 * (nangila_ddp/include/nangila_ffi.h, nangila-hook/src/ffi.rs:27-35, :50-309, :329-457, :848-884).
 * The symbols are exported by nangila/_C*.so. */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* NangilaHandle;

#define NANGILA_DTYPE_FLOAT32 0
#define NANGILA_DTYPE_FLOAT16 1
#define NANGILA_DTYPE_BFLOAT16 2

#define NANGILA_SUCCESS 0
#define NANGILA_INVALID_POINTER 1
#define NANGILA_INVALID_PATH 2
#define NANGILA_IO_ERROR 3
#define NANGILA_COMPRESSION_ERROR 4
#define NANGILA_DECOMPRESSION_ERROR 5

NangilaHandle nangila_init(const char* mask_path);
NangilaHandle nangila_init_all_drivers(uint32_t num_layers);
/* Extension: all-driver hook with explicit warm-up lengths (the reference always uses 1000 + 100). */
NangilaHandle nangila_init_all_drivers_ex(uint32_t num_layers, uint64_t warmup_steps, uint64_t shadow_run_steps);
void nangila_free(NangilaHandle handle);
void nangila_set_gpu_mode(NangilaHandle handle, int32_t enabled);

int32_t nangila_compress(NangilaHandle handle, const float* sendbuff, size_t count, uint32_t layer_id,
                         uint8_t* out_compressed, size_t* out_compressed_size);
int32_t nangila_decompress(NangilaHandle handle, const uint8_t* compressed, size_t compressed_size, uint32_t layer_id,
                           float* recvbuff, size_t count);
int32_t nangila_compress_ex(NangilaHandle handle, const uint8_t* sendbuff, size_t count, int32_t dtype, uint32_t layer_id,
                            uint8_t* out_compressed, size_t* out_compressed_size);
int32_t nangila_decompress_ex(NangilaHandle handle, const uint8_t* compressed, size_t compressed_size, uint32_t layer_id,
                              uint8_t* recvbuff, size_t count, int32_t dtype);
int32_t nangila_on_complete(NangilaHandle handle, const float* gradient, size_t count, uint32_t layer_id);
int32_t nangila_step(NangilaHandle handle);
int32_t nangila_is_enabled(NangilaHandle handle);
uint64_t nangila_current_step(NangilaHandle handle);
uint64_t nangila_predictor_hash(NangilaHandle handle);
/* Upper bound of a packet for `count` FP32 values: 16 + 12 + 4 * count + 32. */
size_t nangila_max_compressed_size(size_t count);

/* ---- tensors that live on the GPU (reference: ffi.rs:526-840; argument order kept) ----------------------------
 * The caller owns the two-step history (`g_current`, `g_previous`: FP32 device buffers of `count` elements) and
 * updates it after the all-reduce, as with the reference. The kernels come from libnangila_kernels.so, bound
 * at the first call (it sits next to this module; NANGILA_KERNELS_LIB overrides); without it the calls return
 * an error code.
 *
 * compress: writes the payload (host wire format: block-64 scales, gain derived on the device) to
 * `out_compressed_payload` (device, 4-byte aligned, nangila_gpu_payload_size(count) bytes) and the 32-byte packet
 * header, with the payload's CRC32, to `out_header_cpu` (host). `*out_compressed_size` = 32 + payload bytes.
 * `scratch_ptr`: 4 bytes of device memory. The call ends with a stream synchronisation (the checksum has to reach
 * the host header). Payloads above 64 MiB (the fixed size of the checksum kernel's device table) are refused.
 * decompress: `compressed` is the whole packet in device memory (header, then payload). Header and checksum are
 * verified before anything is launched (sync_mode 0 skips the checksum); sync_mode 1 also waits for the kernel. */
size_t nangila_gpu_payload_size(size_t count);
int32_t nangila_compress_gpu(NangilaHandle handle, const float* gradient, const float* g_current, const float* g_previous,
                             size_t count, uint32_t layer_id, uint8_t* out_compressed_payload, size_t* out_compressed_size,
                             uint8_t* out_header_cpu, void* stream, uint32_t* scratch_ptr, int32_t sync_mode);
int32_t nangila_decompress_gpu(NangilaHandle handle, const uint8_t* compressed, size_t compressed_size,
                               const float* g_current, const float* g_previous, uint32_t layer_id, float* recvbuff,
                               size_t count, void* stream, uint32_t* scratch_ptr, int32_t sync_mode);

void nangila_enable_safe_mode(NangilaHandle handle, float divergence_threshold, size_t check_interval,
                              uint32_t max_consecutive_failures, size_t recovery_cooldown);
/* 0 Continue, 1 TriggerFallback, 2 RecoveryComplete, 3 NoCheck, 4 CanaryTest */
int32_t nangila_report_val_loss(NangilaHandle handle, float loss);

#ifdef __cplusplus
}
#endif
