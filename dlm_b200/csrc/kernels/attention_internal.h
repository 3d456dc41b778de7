// Kernels behind dlmk::attention (see api.h for the meaning of the arguments).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace dlmk {

// How a score is made from a dot product: dot * scale - slopes[query head] * (query position - key position);
// slopes == nullptr: no distance term.  Converts from a plain scale.
// chunk > 0: a query at p sees only keys j >= floor(p / chunk) * chunk (chunks are counted from position 0 of the
// request).  sinks (f32 [nh], made at load) != nullptr: the softmax's denominator also holds exp(sinks[head]), a
// logit without key or value that is not scaled.
// softcap c > 0: the scaled dot product is squashed, c * tanh(dot * scale / c), before the distance term and the
// mask; 0: it is used as it is.
struct Score {
    float scale;
    const float* slopes;
    int chunk;
    const float* sinks;
    float softcap;
    Score(float s, const float* b = nullptr, int c = 0, const float* k = nullptr, float cap = 0.f)
        : scale(s), slopes(b), chunk(c), sinks(k), softcap(cap) {}
    bool plain_mask() const { return chunk <= 0 && sinks == nullptr; }
    // what the tensor-core kernels get: a squashed score in base-2 units is cap_out() * tanh(dot * cap_in())
    float cap_in() const { return softcap > 0.f ? scale / softcap : 0.f; }
    float cap_out() const { return softcap > 0.f ? softcap * 1.4426950408889634f : 0.f; }
};

#ifdef __CUDACC__
// tanh(x) = 1 - 2 / (2^(2 x log2 e) + 1) on the special-function unit: an absolute error of a few 1e-7 everywhere
// (the scores it squashes are then multiplied by a cap of tens at most), +-1 beyond the range of 2^x.
__device__ __forceinline__ float tanh_sfu(float x) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 2.8853900817779268f));
    return 1.0f - __fdividef(2.0f, e + 1.0f);
}
#endif

// Which of the faster kernels take a chunked mask or a sink: the warp-level prefill kernel and every decode kernel
// do; the tcgen05 prefill kernel does not (its steps go to the warp-level kernel then).
inline bool attention_prefill_takes(const Score&) { return true; }
inline bool attention_decode_takes(const Score&, int /*dtype*/, int /*hd*/) { return true; }

// FMA-unit kernel for any mix of query lengths.  skip_single != 0: requests with exactly one query token are
// left to the decode kernel.
void attention_simt(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                    int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh,
                    int nkv, int hd, int page_size, int total_pages, int window, Score scale, int skip_single,
                    int dtype, cudaStream_t stream);

// Tensor-core kernel (bfloat16) for the head sizes attention_prefill_ok names.
bool attention_prefill_ok(int hd);
void attention_prefill(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                       int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh,
                       int nkv, int hd, int page_size, int total_pages, int window, Score scale, int skip_single,
                       cudaStream_t stream);

// The same on the fifth-generation tensor cores (tcgen05, TMA): head size 128, pages of a power of two of at
// least 64 tokens.  attention_prefill_tc returns false when the tensor maps cannot be made (the caller then
// takes another kernel).  Off with DLM_B200_NO_TCGEN05=1.
bool attention_prefill_tc_enabled();
bool attention_prefill_tc_ok(const void* q, const void* k_cache, const void* v_cache, int nh, int nkv, int hd,
                             int page_size, Score scale);
bool attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                          int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh,
                          int nkv, int hd, int page_size, int total_pages, int window, Score scale, int skip_single,
                          cudaStream_t stream);

// Split-key decode kernel for requests with exactly one query token (bfloat16 and float32).
bool attention_decode_ok(int hd);
void attention_decode_plan(int R, int nkv, int max_kv_len, int* n_splits, int* chunk);
size_t attention_decode_scratch_floats(int R, int nh, int hd, int n_splits);
void attention_decode(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                      int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, float* scratch, int R,
                      int nh, int nkv, int hd, int page_size, int total_pages, int window, Score scale, int n_splits,
                      int chunk, int dtype, cudaStream_t stream);

void attention_decode_merge(const float* part_o, const float* part_ml, const int32_t* cu_q, void* out, int R, int nh,
                            int hd, int n_splits, const float* sinks, int dtype, cudaStream_t stream);
// The same on the tensor-core path (bfloat16, head sizes of attention_prefill_ok); same scratch, same plan.
void attention_decode_mma(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table,
                          int table_width, const int32_t* cu_q, const int32_t* kv_len, void* out, float* scratch,
                          int R, int nh, int nkv, int hd, int page_size, int total_pages, int window, Score scale,
                          int n_splits, int chunk, cudaStream_t stream);

}  // namespace dlmk
