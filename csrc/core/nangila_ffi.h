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

void nangila_enable_safe_mode(NangilaHandle handle, float divergence_threshold, size_t check_interval,
                              uint32_t max_consecutive_failures, size_t recovery_cooldown);
/* 0 Continue, 1 TriggerFallback, 2 RecoveryComplete, 3 NoCheck, 4 CanaryTest */
int32_t nangila_report_val_loss(NangilaHandle handle, float loss);

#ifdef __cplusplus
}
#endif
