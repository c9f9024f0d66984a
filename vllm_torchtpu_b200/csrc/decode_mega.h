// C entry points of the persistent decode kernel (decode_mega.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// size of one per-layer descriptor (tensor maps of the four weight matrices + pointers)
int b200_mega_layer_desc_bytes(void);
// largest number of token rows of a step
int b200_mega_max_tokens(void);
// split-K scratch (bytes) for the per-rank shapes
size_t b200_mega_partial_bytes(int H, int Hq, int Hkv, int I, int num_sms);
int b200_mega_fill_layer(void* desc_host, const void* w_qkv, int n_qkv, int ld_qkv, const void* w_o, int k_o,
                         int ld_o, const void* w_gu, int i2, int ld_gu, const void* w_down, int k_down, int ld_down,
                         int H, const void* ln_in, const void* ln_post, const void* qkv_bias, const void* q_norm,
                         const void* k_norm, void* kv_cache);
int b200_mega_decode(const void* layers_dev, int num_layers, const void* hidden0, void* residual, void* h, void* o,
                     void* act, void* part, size_t part_bytes, const int* positions, const int* slot_mapping,
                     const int* block_tables, const int* seq_lens, int max_blocks, int block_size,
                     long long num_blocks, int T, int H, int Hq, int Hkv, int I, const float* inv_freq,
                     int rot_pairs, int interleaved, float eps, float scale, int kv_splits, void* attn_part_o,
                     void* attn_part_ml, int* attn_counters, int* ctrl, int* status, int world, int rank,
                     void* const* peers, unsigned long long slab0_off, unsigned long long slab1_off,
                     unsigned long long flag0_off, unsigned long long flag1_off, unsigned int spin_limit,
                     int num_sms, unsigned long long* dbg, int dbg_layer, int dbg_gi, int dbg_ev_base,
                     cudaStream_t stream);

#ifdef __cplusplus
}
#endif
