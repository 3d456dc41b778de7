// Small kernels of layers that squash instead of norming: a norm without statistics, tanh(alpha x) w + b; a cap
// c tanh(x / c) on rows of logits; a gate per output entry on attention heads stored wider than their values.
//
// None of these kernels waits on another.  They are launched in the ordinary way (each starts when the kernel before
// it has ended); dep_wait() and dep_launch_next() at their start then do nothing.  The one design that uses them so
// far runs all its steps without programmatic dependent launch (see its model file), and these kernels have not been
// run in a dependent chain since.
#include "api.h"
#include "common.cuh"

namespace dlmk {
namespace {

// An ordinary launch: the kernel starts when the one before it has ended.
template <typename... P, typename... A>
inline void launch_plain(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    kernel<<<grid, block, smem, stream>>>(std::forward<A>(args)...);
}

__device__ __forceinline__ float sigmoid_c(float z) { return 1.0f / (1.0f + expf(-z)); }

// out[i, :] = tanh(alpha * x[rows ? rows[i] : i, :]) * w + b.  TWO: the same rows through a second weight and bias
// into a second output, and with out32 != nullptr that second result once more in 32-bit (one read of x for all).
template <typename T, bool TWO>
__global__ void dyt_norm_kernel(const float* x, const int32_t* __restrict__ rows, const float* __restrict__ w,
                                const float* __restrict__ b, float alpha, T* out, const float* __restrict__ w2,
                                const float* __restrict__ b2, float alpha2, T* out2, float* out32, int H) {
    dep_wait();
    dep_launch_next();
    const long long src = (rows != nullptr ? (long long)rows[blockIdx.x] : (long long)blockIdx.x) * H;
    const long long dst = (long long)blockIdx.x * H;
    constexpr int U = 4;
    for (int i0 = threadIdx.x; i0 < H; i0 += U * blockDim.x) {
        float v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * blockDim.x;
            v[u] = i < H ? x[src + i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * blockDim.x;
            if (i >= H) continue;
            out[dst + i] = from_f32<T>(fmaf(tanhf(alpha * v[u]), w[i], b[i]));
            if (TWO) {
                const float y = fmaf(tanhf(alpha2 * v[u]), w2[i], b2[i]);
                out2[dst + i] = from_f32<T>(y);
                if (out32 != nullptr) out32[dst + i] = y;
            }
        }
    }
}

// x[r, c] = cap * tanh(x[r, c] / cap), in place
__global__ void tanh_cap_kernel(float* x, long long n, float cap, float inv_cap) {
    dep_wait();
    dep_launch_next();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv_cap);
}

// o[t, h * D + i] *= factor * sigmoid(gate[t * ldg + h * dv + i]) for i < dv, in place (entries from dv on are the
// padding of a head stored wider than its values and stay as they are); with resid != nullptr also
// resid[t, :] += bias[:] (W entries): the bias of the projection that follows, added by the launch that is there anyway
template <typename T>
__global__ void entry_gate_kernel(T* o, const float* gate, int ldg, int nh, int dv, int D, float factor, float* resid,
                                  const float* __restrict__ bias, int W) {
    dep_wait();
    dep_launch_next();
    const int t = blockIdx.x;
    if (resid != nullptr)                                  // the output projection's bias joins the token's residual row
        for (int i = threadIdx.x; i < W; i += blockDim.x) resid[(long long)t * W + i] += bias[i];
    T* row = o + (long long)t * nh * D;
    const float* g = gate + (long long)t * ldg;
    constexpr int U = 4;
    const int n = nh * dv;
    for (int i0 = threadIdx.x; i0 < n; i0 += U * blockDim.x) {
        float gv[U], v[U];
        int at[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = i0 + u * blockDim.x;
            at[u] = idx < n ? (idx / dv) * D + idx % dv : 0;
            gv[u] = idx < n ? g[idx] : 0.f;
            v[u] = idx < n ? to_f32(row[at[u]]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (i0 + u * blockDim.x < n) row[at[u]] = from_f32<T>(v[u] * (factor * sigmoid_c(gv[u])));
    }
}

}  // namespace

void dyt_norm(const float* x, const int32_t* rows, const float* w, const float* b, float alpha, void* out, int n_rows,
              int H, int out_dtype, cudaStream_t stream) {
    if (n_rows <= 0) return;
    const dim3 block(H >= 1024 ? 256 : 128);
    if (out_dtype == F32)
        launch_plain(dyt_norm_kernel<float, false>, dim3(n_rows), block, 0, stream, x, rows, w, b, alpha,
                   static_cast<float*>(out), (const float*)nullptr, (const float*)nullptr, 0.f, (float*)nullptr,
                   (float*)nullptr, H);
    else
        launch_plain(dyt_norm_kernel<__nv_bfloat16, false>, dim3(n_rows), block, 0, stream, x, rows, w, b, alpha,
                   static_cast<__nv_bfloat16*>(out), (const float*)nullptr, (const float*)nullptr, 0.f,
                   (__nv_bfloat16*)nullptr, (float*)nullptr, H);
    check_launch("dyt_norm");
}

void dyt_norm_pair(const float* x, const float* wa, const float* ba, float alpha_a, void* out_a, const float* wb,
                   const float* bb, float alpha_b, void* out_b, float* out_b32, int T, int H, int out_dtype,
                   cudaStream_t stream) {
    if (T <= 0) return;
    const dim3 block(H >= 1024 ? 256 : 128);
    if (out_dtype == F32)
        launch_plain(dyt_norm_kernel<float, true>, dim3(T), block, 0, stream, x, (const int32_t*)nullptr, wa, ba, alpha_a,
                   static_cast<float*>(out_a), wb, bb, alpha_b, static_cast<float*>(out_b), out_b32, H);
    else
        launch_plain(dyt_norm_kernel<__nv_bfloat16, true>, dim3(T), block, 0, stream, x, (const int32_t*)nullptr, wa, ba,
                   alpha_a, static_cast<__nv_bfloat16*>(out_a), wb, bb, alpha_b, static_cast<__nv_bfloat16*>(out_b),
                   out_b32, H);
    check_launch("dyt_norm_pair");
}

void tanh_cap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return;
    DLM_CHECK(cap > 0.f, "tanh_cap: the cap must be positive");
    long long blocks = (n + 255) / 256;
    if (blocks > 8LL * sm_count()) blocks = 8LL * sm_count();
    launch_plain(tanh_cap_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, n, cap, 1.0f / cap);
    check_launch("tanh_cap");
}

void entry_gate(void* o, const float* gate, int ldg, int T, int nh, int dv, int D, float factor, int dtype,
                float* resid, const float* bias, int W, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(D >= dv && dv >= 1, "entry_gate: the stored head size must hold the values");
    DLM_CHECK(resid == nullptr || (bias != nullptr && W > 0), "entry_gate: a residual to add to needs the bias and its width");
    if (dtype == F32)
        launch_plain(entry_gate_kernel<float>, dim3(T), dim3(256), 0, stream, static_cast<float*>(o), gate, ldg, nh, dv, D,
                   factor, resid, bias, W);
    else
        launch_plain(entry_gate_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, static_cast<__nv_bfloat16*>(o), gate,
                   ldg, nh, dv, D, factor, resid, bias, W);
    check_launch("entry_gate");
}

}  // namespace dlmk
