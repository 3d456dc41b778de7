// Kernels of the sequence mixers that keep a state per request instead of keys and values, and of the small
// pieces around them: learned positions, several residual streams (hyper-connections), causal convolutions
// over time with their carried inputs, gated group norms, the state-space scan and the delta-rule scan,
// the table that chooses a token's experts, element-wise activations.
//
// Everything here is computed in 32-bit whatever the activation dtype is; only what a kernel hands to a matrix
// product is rounded to the activation dtype.  Every result of a token depends on the tokens before it in its
// own request only, in an order that does not depend on how the request was cut into steps.
#include "api.h"
#include "common.cuh"

namespace dlmk {
namespace {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 30.0f ? z : log1pf(expf(z)); }

template <typename T> __device__ __forceinline__ void put(void* base, long long i, float v) {
    static_cast<T*>(base)[i] = from_f32<T>(v);
}

// --------------------------------------------------------------- learned positions
template <typename T>
__global__ void add_rows_kernel(float* x, const T* __restrict__ table, const int32_t* __restrict__ idx, int H, int rows,
                                int* err) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    const int t = blockIdx.x;
    const int r = idx[t];
    if (r < 0 || r >= rows) {
        if (threadIdx.x == 0) *err = 6;
        return;
    }
    const T* row = table + (long long)r * H;
    float* o = x + (long long)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] += to_f32(row[i]);
}

// ----------------------------------------------------------------- residual streams
__global__ void streams_expand_kernel(const float* __restrict__ x, float* xs, int S, int H) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    const int t = blockIdx.x;
    const float* r = x + (long long)t * H;
    float* o = xs + (long long)t * S * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = r[i];
        for (int s = 0; s < S; ++s) o[(long long)s * H + i] = v;
    }
}

// u = sum_s a[s] xs[t, s, :] (a == nullptr: plain sum); with norm_w: out = u / sqrt(mean(u^2) + eps) * norm_w.
// One block a token; u is kept in shared memory between the two passes.  The sum of squares is added in a fixed
// order: per-thread partial sums over i = tid, tid + 256, ..., a shuffle tree per warp, the warps in order.
template <typename TOut>
__global__ void streams_reduce_kernel(const float* __restrict__ xs, const float* __restrict__ a,
                                      const float* __restrict__ norm_w, float eps, TOut* out, int S, int H) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    extern __shared__ float su[];        // [H]
    __shared__ float s_part[32];
    const int t = blockIdx.x;
    const float* r = xs + (long long)t * S * H;
    float part = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float u = 0.f;
        for (int s = 0; s < S; ++s) u = fmaf(a ? a[s] : 1.0f, r[(long long)s * H + i], u);
        su[i] = u;
        part = fmaf(u, u, part);
    }
    TOut* o = out + (long long)t * H;
    if (norm_w == nullptr) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TOut>(su[i]);
        return;
    }
    const float ss = block_sum(part, s_part);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TOut>((su[i] * inv) * norm_w[i]);
}

// xs[t, r, :] <- sum_s mix[s, r] xs[t, s, :] + outw[r] * y[t, :], all streams at once from the old ones.
// SC: the number of streams at compile time (every loop unrolled, the old values in registers).  blockIdx.y cuts
// a long row into slices so that a step of few tokens still fills the machine.
constexpr int MAX_STREAMS = 16;
template <int SC>
__global__ void streams_update_kernel(float* xs, const float* __restrict__ mix, const float* __restrict__ outw,
                                      const float* __restrict__ y, int H) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    __shared__ float s_mix[SC * SC], s_out[SC];
    for (int i = threadIdx.x; i < SC * SC; i += blockDim.x) s_mix[i] = mix[i];
    for (int i = threadIdx.x; i < SC; i += blockDim.x) s_out[i] = outw[i];
    __syncthreads();
    const int t = blockIdx.x;
    float* r = xs + (long long)t * SC * H;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
        float old[SC];
#pragma unroll
        for (int s = 0; s < SC; ++s) old[s] = r[(long long)s * H + i];
        const float yv = y[(long long)t * H + i];
#pragma unroll
        for (int d = 0; d < SC; ++d) {
            float v = 0.f;
#pragma unroll
            for (int s = 0; s < SC; ++s) v = fmaf(s_mix[s * SC + d], old[s], v);
            r[(long long)d * H + i] = fmaf(s_out[d], yv, v);
        }
    }
}

// The update of one sublayer and the read of the next in one pass over the streams: xs is updated as above, and
// out = rmsnorm(sum_r in_next[r] xs_new[t, r, :]) * norm_w (norm_w == nullptr: the sum itself).  One block a token.
template <int SC, typename TOut>
__global__ void streams_update_reduce_kernel(float* xs, const float* __restrict__ mix, const float* __restrict__ outw,
                                             const float* __restrict__ y, const float* __restrict__ in_next,
                                             const float* __restrict__ norm_w, float eps, TOut* out, int H) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    extern __shared__ float su[];        // [H]
    __shared__ float s_mix[SC * SC], s_out[SC], s_in[SC], s_part[32];
    for (int i = threadIdx.x; i < SC * SC; i += blockDim.x) s_mix[i] = mix[i];
    for (int i = threadIdx.x; i < SC; i += blockDim.x) {
        s_out[i] = outw[i];
        s_in[i] = in_next[i];
    }
    __syncthreads();
    const int t = blockIdx.x;
    float* r = xs + (long long)t * SC * H;
    float part = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float old[SC];
#pragma unroll
        for (int s = 0; s < SC; ++s) old[s] = r[(long long)s * H + i];
        const float yv = y[(long long)t * H + i];
        float u = 0.f;
#pragma unroll
        for (int d = 0; d < SC; ++d) {
            float v = 0.f;
#pragma unroll
            for (int s = 0; s < SC; ++s) v = fmaf(s_mix[s * SC + d], old[s], v);
            v = fmaf(s_out[d], yv, v);
            r[(long long)d * H + i] = v;
            u = fmaf(s_in[d], v, u);
        }
        su[i] = u;
        part = fmaf(u, u, part);
    }
    TOut* o = out + (long long)t * H;
    if (norm_w == nullptr) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TOut>(su[i]);
        return;
    }
    const float ss = block_sum(part, s_part);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TOut>((su[i] * inv) * norm_w[i]);
}

// ------------------------------------------------------------- causal convolution
// out[t, c] = (add_input ? x[t, c] : 0) + bias[c] + sum_j w[c, j] * x[t - taps + 1 + j, c], optionally through silu.
// Inputs before the first token of this step come from the request's carried inputs, state[slot, taps - 1, C]
// (oldest first; zeros when the request starts).
template <typename TOut>
__global__ void causal_conv_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w,
                                   const float* __restrict__ bias, const float* __restrict__ state,
                                   const int32_t* __restrict__ cu_q, const int32_t* __restrict__ token_req,
                                   const int32_t* __restrict__ state_slot, int C, int taps, int add_input, int act,
                                   TOut* out, int ldo) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    const int t = blockIdx.x;
    const int r = token_req[t];
    const int start = cu_q[r];
    const long long sbase = (long long)state_slot[r] * (taps - 1) * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float acc = bias ? bias[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = t - (taps - 1) + j;
            const float v = src >= start ? x[(long long)src * ldx + c]
                                         : state[sbase + (long long)((taps - 1) + (src - start)) * C + c];
            acc = fmaf(w[(long long)c * taps + j], v, acc);
        }
        if (add_input) acc += x[(long long)t * ldx + c];
        if (act == 1) acc = silu_f(acc);
        out[(long long)t * ldo + c] = from_f32<TOut>(acc);
    }
}

// The carried inputs after the step: the last taps - 1 of (old carried inputs, this step's inputs).  One thread
// owns a (request, channel): it reads what it needs before it writes.
constexpr int MAX_TAPS = 16;
__global__ void conv_state_kernel(const float* __restrict__ x, int ldx, float* state, const int32_t* __restrict__ cu_q,
                                  const int32_t* __restrict__ state_slot, int C, int taps) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    const int r = blockIdx.x;
    const int start = cu_q[r], n = cu_q[r + 1] - start;
    const int keep = taps - 1;
    float* st = state + (long long)state_slot[r] * keep * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float v[MAX_TAPS];
        for (int i = 0; i < keep; ++i) {
            const int src = n - keep + i;         // index among this step's tokens; negative: an old carried input
            v[i] = src >= 0 ? x[(long long)(start + src) * ldx + c] : st[(long long)(keep + src) * C + c];
        }
        for (int i = 0; i < keep; ++i) st[(long long)i * C + c] = v[i];
    }
}

// -------------------------------------------------------------------- activations
template <typename TOut>
__global__ void activation_kernel(const float* __restrict__ x, int ldx, TOut* out, int ldo, int cols, int op) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    const int r = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < cols; c += gridDim.y * blockDim.x) {
        const float z = x[(long long)r * ldx + c];
        float v;
        switch (op) {
            case 0: v = tanhf(z); break;
            case 1: v = gelu_exact_f(z); break;
            case 2: v = silu_f(z); break;
            case 3: v = gelu_tanh_f(z); break;
            default: v = z; break;          // 4: a copy (a change of format)
        }
        out[(long long)r * ldo + c] = from_f32<TOut>(v);
    }
}

// ------------------------------------------------------------ experts from a table
__global__ void table_lookup_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ table, int32_t* ids,
                                    float* wts, int T, int V, int top, int E, int* err) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * top) return;
    const int t = i / top, j = i - t * top;
    const int tok = tokens[t];
    int e = 0;
    if (tok < 0 || tok >= V) {
        *err = 1;
    } else {
        e = table[(long long)tok * top + j];
        if (e < 0 || e >= E) {
            *err = 4;
            e = 0;
        }
    }
    ids[i] = e;
    wts[i] = 1.0f / (float)top;
}

// ---------------------------------------------------------------- gated group norm
// One block a (token, group) of `gs` channels.  mode 0: v = y * silu(gate); out = v / rms(v) * w.
// mode 1: out = y / rms(y) * w * sigmoid(gate).  rms over the group, eps inside the root.
template <typename TOut>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ y, int ldy, const float* __restrict__ gate, int ldg,
                                     const float* __restrict__ w, TOut* out, int ldo, int gs, float eps, int mode,
                                     const float* row_scale) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    __shared__ float s_part[32];
    const int t = blockIdx.x, g = blockIdx.y;
    const float* yr = y + (long long)t * ldy + (long long)g * gs;
    const float* gr = gate + (long long)t * ldg + (long long)g * gs;
    if (row_scale != nullptr) {
        // y is first multiplied by a factor per (token, group); the norm's eps then meets the scaled values
        const float f = row_scale[(long long)t * gridDim.y + g];
        float part = 0.f;
        for (int i = threadIdx.x; i < gs; i += blockDim.x) {
            const float v = yr[i] * f;
            part = fmaf(v, v, part);
        }
        const float inv = 1.0f / sqrtf(block_sum(part, s_part) / (float)gs + eps);
        TOut* o = out + (long long)t * ldo + (long long)g * gs;
        for (int i = threadIdx.x; i < gs; i += blockDim.x) {
            const float wi = w != nullptr ? w[(long long)g * gs + i] : 1.0f;
            const float v = ((yr[i] * f) * inv) * wi;
            o[i] = from_f32<TOut>(mode == 1 ? v * sigmoid_f(gr[i]) : v * silu_f(gr[i]));
        }
        return;
    }
    float part = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float v = mode == 0 ? yr[i] * silu_f(gr[i]) : yr[i];
        part = fmaf(v, v, part);
    }
    const float ss = block_sum(part, s_part);
    const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
    TOut* o = out + (long long)t * ldo + (long long)g * gs;
    const float* wr = w != nullptr ? w + (long long)g * gs : nullptr;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float wi = wr != nullptr ? wr[i] : 1.0f;
        float v;
        if (mode == 0) v = ((yr[i] * silu_f(gr[i])) * inv) * wi;
        else if (mode == 1) v = ((yr[i] * inv) * wi) * sigmoid_f(gr[i]);
        else v = ((yr[i] * inv) * wi) * silu_f(gr[i]);
        o[i] = from_f32<TOut>(v);
    }
}

// ------------------------------------------------------------ pieces of the two scans
// Four bytes from global to shared memory without a register in between; a group of such copies is waited for
// with copies_wait<N>() (all but the N newest groups have landed).
__device__ __forceinline__ void copy4_async(float* dst_smem, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copy16_async(float* dst_smem, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
template <int N> __device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---------------------------------------------------------------- state-space scan
// Per head: S <- exp(-exp(A_log) dt) S + dt B x^T (S is N x P), y = S^T C + D x, dt = softplus(dt_raw + dt_bias).
// A block owns (head, request, a chunk of the P columns) and walks the request's tokens in order.  Column p of S
// is shared by `parts` neighbouring lanes (a power of two): lane `part` keeps rows part, part + parts, ... in
// registers (NPT of them), adds up its share of S^T C and the shares meet in a butterfly of shuffles, so the order
// of every sum is fixed by (N, parts) alone.  The tokens' inputs come in tiles of `tile` tokens (B, C, the block's
// x columns, dt), copied asynchronously into one of two buffers while the tile before is worked on; within a tile
// nothing waits for memory.
// VEC (N a multiple of 4): a lane's rows come in fours, 4 part + e + 4 parts q, so that B and C are read with
// 16-byte shared loads that neighbouring lanes take from neighbouring addresses.
constexpr int SSM_STAGES = 4;

template <int NPT, bool VEC>
__global__ void ssm_scan_kernel(const float* __restrict__ xbc, int ldx, const float* __restrict__ dt_raw, int lddt,
                                const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                const float* __restrict__ D, float* state, const int32_t* __restrict__ cu_q,
                                const int32_t* __restrict__ state_slot, float* y, int heads, int P, int N, int groups,
                                int parts, int tile, int wide, const float* __restrict__ fixed_decay) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    // (a long kernel, launched in the ordinary way: its blocks are placed when the machine is free, and the
    // kernel after it is let in only when it ends)
    extern __shared__ __align__(16) float sm[];            // [SSM_STAGES][tile][2 N + cols + 2]: B, C, x, dt, decay
    const int h = blockIdx.x, r = blockIdx.y;
    const int cols = blockDim.x / parts;
    const int part = threadIdx.x % parts;
    const int col = threadIdx.x / parts;
    const int p0 = blockIdx.z * cols;
    const int p = p0 + col;
    const bool live = p < P;
    const int g = h / (heads / groups);
    const int inner = heads * P;
    const int rl = (2 * N + cols + 2 + 3) & ~3;
    float* st = state + (((long long)state_slot[r] * heads + h) * N) * P;
    auto row_of = [&](int i) { return VEC ? 4 * part + (i & 3) + 4 * parts * (i >> 2) : part + parts * i; };
    float s[NPT];
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = row_of(i);
        s[i] = (live && n < N) ? st[(long long)n * P + p] : 0.f;
    }
    // fixed_decay: the step size is 1 and the head's decay a constant of the model (dt_raw, dt_bias, A_log unused)
    const bool fixed = fixed_decay != nullptr;
    const float a = fixed ? 0.f : -expf(A_log[h]), dcoef = D != nullptr ? D[h] : 0.f, bias = fixed ? 0.f : dt_bias[h];
    const float decay_h = fixed ? fixed_decay[h] : 0.f;
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    const int n_tiles = (t1 - t0 + tile - 1) / tile;
    // a warp fetches a token at a time; `wide`: every run starts on a 16-byte boundary and is a multiple of four
    auto fetch = [&](int k) {             // (a tile beyond the last: an empty group, so that the count of groups holds)
        float* buf = sm + (size_t)(k % SSM_STAGES) * tile * rl;
        const int first = t0 + k * tile, n = min(tile, t1 - first);
        const int lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
        for (int tok = threadIdx.x >> 5; tok < n; tok += nwarp) {
            const float* row = xbc + (long long)(first + tok) * ldx;
            const float* srcB = row + inner + g * N;
            const float* srcC = row + inner + groups * N + g * N;
            const float* srcX = row + h * P + p0;
            float* dst = buf + (size_t)tok * rl;
            const int nx = min(cols, P - p0);
            if (wide) {
                for (int i = 4 * lane; i < N; i += 128) {
                    copy16_async(dst + i, srcB + i);
                    copy16_async(dst + N + i, srcC + i);
                }
                for (int i = 4 * lane; i < nx; i += 128) copy16_async(dst + 2 * N + i, srcX + i);
            } else {
                for (int i = lane; i < N; i += 32) {
                    copy4_async(dst + i, srcB + i);
                    copy4_async(dst + N + i, srcC + i);
                }
                for (int i = lane; i < nx; i += 32) copy4_async(dst + 2 * N + i, srcX + i);
            }
            if (lane == 0 && !fixed) copy4_async(dst + 2 * N + cols, dt_raw + (long long)(first + tok) * lddt + h);
        }
        copies_commit();
    };
    // tiles are asked for three ahead of the one worked on: a tile's walk is shorter than a trip to memory
    for (int k = 0; k < SSM_STAGES - 1; ++k) fetch(k);
    for (int k = 0; k < n_tiles; ++k) {
        fetch(k + SSM_STAGES - 1);           // into the buffer of tile k - 1, freed by the barrier that ended its walk
        copies_wait<SSM_STAGES - 1>();
        __syncthreads();
        float* buf = sm + (size_t)(k % SSM_STAGES) * tile * rl;
        const int first = t0 + k * tile, n = min(tile, t1 - first);
        if (threadIdx.x < n) {
            float* row = buf + (size_t)threadIdx.x * rl;
            const float dt = fixed ? 1.0f : softplus_f(row[2 * N + cols] + bias);
            row[2 * N + cols] = dt;
            row[2 * N + cols + 1] = fixed ? decay_h : expf(a * dt);
        }
        __syncthreads();
        // (unrolled: a token depends on the one before it through the state's own multiply-add only, so the sums
        // and shuffles of neighbouring tokens overlap)
#pragma unroll 4
        for (int tok = 0; tok < n; ++tok) {
            const float* row = buf + (size_t)tok * rl;
            const float dt = row[2 * N + cols], decay = row[2 * N + cols + 1];
            const float xv = live ? row[2 * N + col] : 0.f;
            const float dx = dt * xv;
            float acc = 0.f;
            if (VEC) {
#pragma unroll
                for (int q = 0; q < NPT / 4; ++q) {
                    const int nn = 4 * part + 4 * parts * q;
                    if (nn < N) {
                        const float4 bv = *reinterpret_cast<const float4*>(row + nn);
                        const float4 cv = *reinterpret_cast<const float4*>(row + N + nn);
                        s[4 * q + 0] = fmaf(decay, s[4 * q + 0], dx * bv.x);
                        s[4 * q + 1] = fmaf(decay, s[4 * q + 1], dx * bv.y);
                        s[4 * q + 2] = fmaf(decay, s[4 * q + 2], dx * bv.z);
                        s[4 * q + 3] = fmaf(decay, s[4 * q + 3], dx * bv.w);
                        acc = fmaf(s[4 * q + 0], cv.x, acc);
                        acc = fmaf(s[4 * q + 1], cv.y, acc);
                        acc = fmaf(s[4 * q + 2], cv.z, acc);
                        acc = fmaf(s[4 * q + 3], cv.w, acc);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < NPT; ++i) {
                    const int nn = part + parts * i;
                    if (nn < N) {
                        s[i] = fmaf(decay, s[i], dx * row[nn]);
                        acc = fmaf(s[i], row[N + nn], acc);
                    }
                }
            }
            for (int o = parts >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && part == 0) y[(long long)(first + tok) * inner + h * P + p] = fmaf(dcoef, xv, acc);
        }
        __syncthreads();                     // the buffer may be filled again
    }
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = row_of(i);
        if (live && n < N) st[(long long)n * P + p] = s[i];
    }
}

// ----------------------------------------------------------------- delta-rule scan
// Per head, with key channels i and value channels j (d of each):
//   w = exp(-decay_coef sigmoid(lw)), a = sigmoid(a_raw + a_bias), u = k / sqrt(sum k^2 + unit_eps)
//   S <- diag(w) S - (a u) (u^T S) + k v^T   (both terms read the old S);   o = S^T r
// A block owns (head, request, a chunk of value columns).  Column j of S is shared by `parts` neighbouring lanes,
// lane `part` keeps rows part, part + parts, ... in registers; sum k^2, u^T S and S^T r are added per lane and
// meet in a butterfly of shuffles (a fixed order).  Inputs come in tiles of `tile` tokens (r, k, raw a, raw w, the
// block's v columns) by asynchronous copies into one of two buffers, as in the state-space scan.
template <int NPT, bool VEC>
__global__ void delta_scan_kernel(const float* __restrict__ proj, int ld, int off_r, int off_k, int off_v, int off_a,
                                  const float* __restrict__ lw, int ldlw, const float* __restrict__ a_bias, float* state,
                                  const int32_t* __restrict__ cu_q, const int32_t* __restrict__ state_slot, float* o,
                                  int heads, int d, float unit_eps, float decay_coef, int parts, int tile, int wide) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    // (a long kernel, launched in the ordinary way: its blocks are placed when the machine is free, and the
    // kernel after it is let in only when it ends)
    extern __shared__ __align__(16) float sm[];            // [2][tile][4 d + cols]: r, k, a, w, v
    const int h = blockIdx.x, r = blockIdx.y;
    const int cols = blockDim.x / parts;
    const int part = threadIdx.x % parts;
    const int col = threadIdx.x / parts;
    const int j0 = blockIdx.z * cols;
    const int j = j0 + col;
    const bool live = j < d;
    const int rl = (4 * d + cols + 3) & ~3;
    float* st = state + (((long long)state_slot[r] * heads + h) * d) * d;
    auto row_of = [&](int ii) { return VEC ? 4 * part + (ii & 3) + 4 * parts * (ii >> 2) : part + parts * ii; };
    float s[NPT];
#pragma unroll
    for (int ii = 0; ii < NPT; ++ii) {
        const int i = row_of(ii);
        s[ii] = (live && i < d) ? st[(long long)i * d + j] : 0.f;
    }
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    const int hd = h * d;
    const int n_tiles = (t1 - t0 + tile - 1) / tile;
    // a warp fetches a token at a time; `wide`: every run starts on a 16-byte boundary and is a multiple of four
    auto fetch = [&](int k) {
        float* buf = sm + (size_t)(k & 1) * tile * rl;
        const int first = t0 + k * tile, n = min(tile, t1 - first);
        const int lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
        for (int tok = threadIdx.x >> 5; tok < n; tok += nwarp) {
            const float* row = proj + (long long)(first + tok) * ld + hd;
            const float* srcW = lw + (long long)(first + tok) * ldlw + hd;
            float* dst = buf + (size_t)tok * rl;
            const int nv = min(cols, d - j0);
            if (wide) {
                for (int i = 4 * lane; i < d; i += 128) {
                    copy16_async(dst + i, row + off_r + i);
                    copy16_async(dst + d + i, row + off_k + i);
                    copy16_async(dst + 2 * d + i, row + off_a + i);
                    copy16_async(dst + 3 * d + i, srcW + i);
                }
                for (int i = 4 * lane; i < nv; i += 128) copy16_async(dst + 4 * d + i, row + off_v + j0 + i);
            } else {
                for (int i = lane; i < d; i += 32) {
                    copy4_async(dst + i, row + off_r + i);
                    copy4_async(dst + d + i, row + off_k + i);
                    copy4_async(dst + 2 * d + i, row + off_a + i);
                    copy4_async(dst + 3 * d + i, srcW + i);
                }
                for (int i = lane; i < nv; i += 32) copy4_async(dst + 4 * d + i, row + off_v + j0 + i);
            }
        }
        copies_commit();
    };
    if (n_tiles > 0) fetch(0);
    for (int k = 0; k < n_tiles; ++k) {
        if (k + 1 < n_tiles) {
            fetch(k + 1);
            copies_wait<1>();
        } else {
            copies_wait<0>();
        }
        __syncthreads();
        float* buf = sm + (size_t)(k & 1) * tile * rl;
        const int first = t0 + k * tile, n = min(tile, t1 - first);
        for (int idx = threadIdx.x; idx < n * d; idx += blockDim.x) {       // raw values -> removal rate and decay
            const int tok = idx / d, i = idx - tok * d;
            float* row = buf + (size_t)tok * rl;
            row[2 * d + i] = sigmoid_f(row[2 * d + i] + a_bias[hd + i]);
            row[3 * d + i] = expf(-decay_coef * sigmoid_f(row[3 * d + i]));
        }
        __syncthreads();
        for (int tok = 0; tok < n; ++tok) {
            const float* br = buf + (size_t)tok * rl;
            const float* bk = br + d;
            const float* ba = br + 2 * d;
            const float* bw = br + 3 * d;
            float ss = 0.f, us = 0.f;
            float kk[NPT], ww[NPT], aa[NPT], rr[NPT];   // this lane's rows of k, w, a, r
#pragma unroll
            for (int ii = 0; ii < NPT; ++ii) kk[ii] = ww[ii] = aa[ii] = rr[ii] = 0.f;
            if (VEC) {
#pragma unroll
                for (int q = 0; q < NPT / 4; ++q) {
                    const int i = 4 * part + 4 * parts * q;
                    if (i < d) {
                        const float4 k4 = *reinterpret_cast<const float4*>(bk + i), w4 = *reinterpret_cast<const float4*>(bw + i);
                        const float4 a4 = *reinterpret_cast<const float4*>(ba + i), r4 = *reinterpret_cast<const float4*>(br + i);
                        kk[4 * q] = k4.x; kk[4 * q + 1] = k4.y; kk[4 * q + 2] = k4.z; kk[4 * q + 3] = k4.w;
                        ww[4 * q] = w4.x; ww[4 * q + 1] = w4.y; ww[4 * q + 2] = w4.z; ww[4 * q + 3] = w4.w;
                        aa[4 * q] = a4.x; aa[4 * q + 1] = a4.y; aa[4 * q + 2] = a4.z; aa[4 * q + 3] = a4.w;
                        rr[4 * q] = r4.x; rr[4 * q + 1] = r4.y; rr[4 * q + 2] = r4.z; rr[4 * q + 3] = r4.w;
                    }
                }
            } else {
#pragma unroll
                for (int ii = 0; ii < NPT; ++ii) {
                    const int i = part + parts * ii;
                    if (i < d) { kk[ii] = bk[i]; ww[ii] = bw[i]; aa[ii] = ba[i]; rr[ii] = br[i]; }
                }
            }
#pragma unroll
            for (int ii = 0; ii < NPT; ++ii) {          // rows beyond d hold zeros and add nothing
                ss = fmaf(kk[ii], kk[ii], ss);
                us = fmaf(kk[ii], s[ii], us);           // k^T S; scaled to u^T S below
            }
            for (int x = parts >> 1; x > 0; x >>= 1) {
                ss += __shfl_xor_sync(0xffffffffu, ss, x);
                us += __shfl_xor_sync(0xffffffffu, us, x);
            }
            const float inv = 1.0f / sqrtf(ss + unit_eps);
            us *= inv;
            const float vj = live ? br[4 * d + col] : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int ii = 0; ii < NPT; ++ii) {
                float v = ww[ii] * s[ii];
                v = fmaf(-(aa[ii] * (kk[ii] * inv)), us, v);
                v = fmaf(kk[ii], vj, v);
                s[ii] = v;
                acc = fmaf(v, rr[ii], acc);
            }
            for (int x = parts >> 1; x > 0; x >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, x);
            if (live && part == 0) o[(long long)(first + tok) * heads * d + hd + j] = acc;
        }
        __syncthreads();                     // the buffer may be filled again
    }
#pragma unroll
    for (int ii = 0; ii < NPT; ++ii) {
        const int i = row_of(ii);
        if (live && i < d) st[(long long)i * d + j] = s[ii];
    }
}

// Tokens a tile of a scan: 16, fewer when a token's inputs are so wide that two buffers of 16 would not fit.
int scan_tile(int row_floats) {
    int t = 16;
    while (t > 1 && 2 * (size_t)t * row_floats * sizeof(float) > 96 * 1024) t /= 2;
    return t;
}

// How a column's rows are dealt to lanes: `parts` lanes (a power of two, at most 32) with at most `per` rows each.
void scan_layout(int rows, int width, int per, int* parts, int* cols, int* chunks, bool vec = false) {
    int pt = 1;
    if (vec) {                                              // rows are dealt in fours
        const int quads = rows / 4, per_q = per / 4;
        while (pt < 32 && (quads + pt - 1) / pt > per_q) pt *= 2;
    } else {
        while (pt < 32 && (rows + pt - 1) / pt > per) pt *= 2;
    }
    const int unit = 32 / pt;                               // columns a warp holds
    int c = ((width + unit - 1) / unit) * unit;
    if (c > 256 / pt) c = 256 / pt;
    *parts = pt;
    *cols = c;
    *chunks = (width + c - 1) / c;
}

}  // namespace

// ======================================================================= launchers
void add_rows(float* x, const void* table, const int32_t* idx, int T, int H, int rows, int dtype, cudaStream_t stream) {
    if (T <= 0) return;
    int* err = error_flag_ptr();
    if (dtype == F32) launch_dep(add_rows_kernel<float>, dim3(T), dim3(256), 0, stream, x, static_cast<const float*>(table), idx, H, rows, err);
    else launch_dep(add_rows_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, x, static_cast<const __nv_bfloat16*>(table), idx, H, rows, err);
    check_launch("add_rows");
}

void streams_expand(const float* x, float* xs, int T, int S, int H, cudaStream_t stream) {
    if (T <= 0) return;
    launch_dep(streams_expand_kernel, dim3(T), dim3(256), 0, stream, x, xs, S, H);
    check_launch("streams_expand");
}

void streams_reduce(const float* xs, const float* a, const float* norm_w, float eps, void* out, int T, int S, int H,
                    int out_dtype, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(S >= 1 && H >= 1, "streams_reduce: sizes");
    const size_t smem = (size_t)H * sizeof(float);
    DLM_CHECK(smem <= 200 * 1024, "streams_reduce: a row does not fit in shared memory");
    if (out_dtype == F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_reduce_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dep(streams_reduce_kernel<float>, dim3(T), dim3(256), smem, stream, xs, a, norm_w, eps, static_cast<float*>(out), S, H);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_reduce_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dep(streams_reduce_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, stream, xs, a, norm_w, eps, static_cast<__nv_bfloat16*>(out), S, H);
    }
    check_launch("streams_reduce");
}

void streams_update(float* xs, const float* mix, const float* outw, const float* y, int T, int S, int H,
                    cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(S >= 1 && S <= MAX_STREAMS, "streams_update: at most 16 residual streams");
    const int slices = T >= 2 * sm_count() ? 1 : (H + 255) / 256;
    const dim3 grid(T, slices);
    switch (S) {
#define DLM_SU(N) case N: launch_dep(streams_update_kernel<N>, dim3(grid), dim3(256), 0, stream, xs, mix, outw, y, H); break;
        DLM_SU(1) DLM_SU(2) DLM_SU(3) DLM_SU(4) DLM_SU(5) DLM_SU(6) DLM_SU(7) DLM_SU(8) DLM_SU(9) DLM_SU(10) DLM_SU(11)
        DLM_SU(12) DLM_SU(13) DLM_SU(14) DLM_SU(15) DLM_SU(16)
#undef DLM_SU
    }
    check_launch("streams_update");
}

namespace {
template <int SC>
void launch_update_reduce(float* xs, const float* mix, const float* outw, const float* y, const float* in_next,
                          const float* norm_w, float eps, void* out, int T, int H, int out_dtype, cudaStream_t stream) {
    const size_t smem = (size_t)H * sizeof(float);
    if (out_dtype == F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(streams_update_reduce_kernel<SC, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dep(streams_update_reduce_kernel<SC, float>, dim3(T), dim3(256), smem, stream, xs, mix, outw, y, in_next,
                   norm_w, eps, static_cast<float*>(out), H);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(streams_update_reduce_kernel<SC, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_dep(streams_update_reduce_kernel<SC, __nv_bfloat16>, dim3(T), dim3(256), smem, stream, xs, mix, outw, y,
                   in_next, norm_w, eps, static_cast<__nv_bfloat16*>(out), H);
    }
}
}  // namespace

void streams_update_reduce(float* xs, const float* mix, const float* outw, const float* y, const float* in_next,
                           const float* norm_w, float eps, void* out, int T, int S, int H, int out_dtype,
                           cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(S >= 1 && S <= 8, "streams_update_reduce: at most 8 residual streams");
    DLM_CHECK((size_t)H * sizeof(float) <= 200 * 1024, "streams_update_reduce: a row does not fit in shared memory");
    switch (S) {
#define DLM_SUR(N) case N: launch_update_reduce<N>(xs, mix, outw, y, in_next, norm_w, eps, out, T, H, out_dtype, stream); break;
        DLM_SUR(1) DLM_SUR(2) DLM_SUR(3) DLM_SUR(4) DLM_SUR(5) DLM_SUR(6) DLM_SUR(7) DLM_SUR(8)
#undef DLM_SUR
    }
    check_launch("streams_update_reduce");
}

void causal_conv(const float* x, int ldx, const float* w, const float* bias, float* state, const int32_t* cu_q,
                 const int32_t* token_req, const int32_t* state_slot, int T, int R, int C, int taps, int add_input,
                 int act, void* out, int ldo, int out_dtype, cudaStream_t stream) {
    if (T <= 0 || R <= 0) return;
    DLM_CHECK(taps >= 1 && taps <= MAX_TAPS, "causal_conv: 1 to 16 taps");
    const int slices = (C + 255) / 256;
    if (out_dtype == F32)
        launch_dep(causal_conv_kernel<float>, dim3(T, slices), dim3(256), 0, stream, x, ldx, w, bias, state, cu_q, token_req, state_slot,
                                                                    C, taps, add_input, act, static_cast<float*>(out), ldo);
    else
        launch_dep(causal_conv_kernel<__nv_bfloat16>, dim3(T, slices), dim3(256), 0, stream, 
            x, ldx, w, bias, state, cu_q, token_req, state_slot, C, taps, add_input, act,
            static_cast<__nv_bfloat16*>(out), ldo);
    check_launch("causal_conv");
    if (taps > 1) {
        launch_dep(conv_state_kernel, dim3(R, slices), dim3(256), 0, stream, x, ldx, state, cu_q, state_slot, C, taps);
        check_launch("conv_state");
    }
}

void activation(const float* x, int ldx, void* out, int ldo, int rows, int cols, int op, int out_dtype,
                cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return;
    const int slices = (cols + 255) / 256 > 64 ? 64 : (cols + 255) / 256;
    if (out_dtype == F32)
        launch_dep(activation_kernel<float>, dim3(rows, slices), dim3(256), 0, stream, x, ldx, static_cast<float*>(out), ldo, cols, op);
    else
        launch_dep(activation_kernel<__nv_bfloat16>, dim3(rows, slices), dim3(256), 0, stream, x, ldx, static_cast<__nv_bfloat16*>(out),
                                                                              ldo, cols, op);
    check_launch("activation");
}

void table_lookup(const int32_t* tokens, const int32_t* table, int32_t* ids, float* wts, int T, int V, int top, int E,
                  cudaStream_t stream) {
    if (T <= 0) return;
    const int n = T * top;
    launch_dep(table_lookup_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, tokens, table, ids, wts, T, V, top, E, error_flag_ptr());
    check_launch("table_lookup");
}

void gated_rmsnorm(const float* y, int ldy, const float* gate, int ldg, const float* w, void* out, int ldo, int T,
                   int groups, int group_size, float eps, int mode, int out_dtype, const float* row_scale,
                   cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(row_scale == nullptr || mode != 0, "gated_rmsnorm: a factor per row goes with a gate after the norm");
    const int threads = group_size >= 256 ? 256 : (group_size >= 128 ? 128 : (group_size > 32 ? 64 : 32));
    if (out_dtype == F32)
        launch_dep(gated_rmsnorm_kernel<float>, dim3(T, groups), dim3(threads), 0, stream, y, ldy, gate, ldg, w, static_cast<float*>(out),
                                                                          ldo, group_size, eps, mode, row_scale);
    else
        launch_dep(gated_rmsnorm_kernel<__nv_bfloat16>, dim3(T, groups), dim3(threads), 0, stream, 
            y, ldy, gate, ldg, w, static_cast<__nv_bfloat16*>(out), ldo, group_size, eps, mode, row_scale);
    check_launch("gated_rmsnorm");
}

void ssm_scan(const float* xbc, int ldx, const float* dt_raw, int lddt, const float* dt_bias, const float* A_log,
              const float* D, float* state, const int32_t* cu_q, const int32_t* state_slot, float* y, int R, int heads,
              int P, int N, int groups, const float* fixed_decay, cudaStream_t stream) {
    if (R <= 0) return;
    DLM_CHECK(fixed_decay != nullptr || (dt_raw != nullptr && dt_bias != nullptr && A_log != nullptr && D != nullptr),
              "ssm_scan: without fixed decays the step sizes, their bias, A_log and D are needed");
    DLM_CHECK(groups >= 1 && heads % groups == 0, "ssm_scan: heads must be a multiple of groups");
    DLM_CHECK(N >= 1 && N <= 1024, "ssm_scan: state size 1..1024");
    int parts, cols, chunks;
    const bool vec = N % 4 == 0;
    scan_layout(N, P, 8, &parts, &cols, &chunks, vec);   // few rows a lane: many lanes a column, many warps an SM
    // a launch that leaves multiprocessors idle (a prompt of one request, few heads): half the rows a lane, twice the blocks
    if (vec && (long long)heads * R * chunks < sm_count()) scan_layout(N, P, 4, &parts, &cols, &chunks, vec);
    const int per = vec ? 4 * ((N / 4 + parts - 1) / parts) : (N + parts - 1) / parts;
    const int rl = (2 * N + cols + 2 + 3) & ~3;
    int tile = scan_tile(rl);
    while (tile > 1 && SSM_STAGES * (size_t)tile * rl * sizeof(float) > 96 * 1024) tile /= 2;
    const size_t smem = SSM_STAGES * (size_t)tile * rl * sizeof(float);
    DLM_CHECK(smem <= 200 * 1024, "ssm_scan: a token's inputs do not fit in shared memory");
    const dim3 grid(heads, R, chunks);
    // 16-byte copies: every run of a token's inputs starts on a 16-byte boundary and is a multiple of four floats
    const int wide = (reinterpret_cast<uintptr_t>(xbc) % 16 == 0 && ldx % 4 == 0 && N % 4 == 0 && P % 4 == 0 &&
                      cols % 4 == 0 && (heads * P) % 4 == 0) ? 1 : 0;
#define DLM_SSM(NPT, V)                                                                                               \
    do {                                                                                                              \
        if (smem > 48 * 1024)                                                                                         \
            cudaFuncSetAttribute(ssm_scan_kernel<NPT, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        ssm_scan_kernel<NPT, V><<<grid, cols * parts, smem, stream>>>(xbc, ldx, dt_raw, lddt, dt_bias, A_log, D, state, \
                                                                     cu_q, state_slot, y, heads, P, N, groups, parts, \
                                                                     tile, wide, fixed_decay);                        \
    } while (0)
    if (vec) {
        if (per <= 4) DLM_SSM(4, true);
        else if (per <= 8) DLM_SSM(8, true);
        else if (per <= 16) DLM_SSM(16, true);
        else DLM_SSM(32, true);
    } else {
        if (per <= 8) DLM_SSM(8, false);
        else if (per <= 16) DLM_SSM(16, false);
        else DLM_SSM(32, false);
    }
#undef DLM_SSM
    check_launch("ssm_scan");
}

void delta_scan(const float* proj, int ld, int off_r, int off_k, int off_v, int off_a, const float* lw, int ldlw,
                const float* a_bias, float* state, const int32_t* cu_q, const int32_t* state_slot, float* o, int R,
                int heads, int d, float unit_eps, float decay_coef, cudaStream_t stream) {
    if (R <= 0) return;
    DLM_CHECK(d >= 1 && d <= 512, "delta_scan: head size 1..512");
    int parts, cols, chunks;
    const bool vec = d % 4 == 0;
    scan_layout(d, d, 4, &parts, &cols, &chunks, vec);
    const int per = vec ? 4 * ((d / 4 + parts - 1) / parts) : (d + parts - 1) / parts;
    const int rl = (4 * d + cols + 3) & ~3;
    const int tile = scan_tile(rl);
    const size_t smem = 2 * (size_t)tile * rl * sizeof(float);
    DLM_CHECK(smem <= 200 * 1024, "delta_scan: a token's inputs do not fit in shared memory");
    const dim3 grid(heads, R, chunks);
    const int wide = (reinterpret_cast<uintptr_t>(proj) % 16 == 0 && reinterpret_cast<uintptr_t>(lw) % 16 == 0 &&
                      ld % 4 == 0 && ldlw % 4 == 0 && d % 4 == 0 && cols % 4 == 0 && off_r % 4 == 0 && off_k % 4 == 0 &&
                      off_v % 4 == 0 && off_a % 4 == 0) ? 1 : 0;
#define DLM_DELTA(NPT, V)                                                                                             \
    do {                                                                                                              \
        if (smem > 48 * 1024)                                                                                         \
            cudaFuncSetAttribute(delta_scan_kernel<NPT, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        delta_scan_kernel<NPT, V><<<grid, cols * parts, smem, stream>>>(proj, ld, off_r, off_k, off_v, off_a, lw, ldlw, \
                                                                       a_bias, state, cu_q, state_slot, o, heads, d,  \
                                                                       unit_eps, decay_coef, parts, tile, wide);      \
    } while (0)
    if (vec) {
        if (per <= 4) DLM_DELTA(4, true);
        else if (per <= 8) DLM_DELTA(8, true);
        else DLM_DELTA(16, true);
    } else {
        if (per <= 4) DLM_DELTA(4, false);
        else if (per <= 8) DLM_DELTA(8, false);
        else DLM_DELTA(16, false);
    }
#undef DLM_DELTA
    check_launch("delta_scan");
}

}  // namespace dlmk
