// Gated recurrences with a matrix state per head, per-head query/key norms with rotary positions and the paged
// write, a gate per head, and the small residual-stream kernels of layers with a norm on both sides of a sublayer.
//
// None of these kernels waits on another (no spin, no mbarrier).  The short ones are launched with programmatic
// dependent launch (dep_wait() is their first statement); the scan is launched in the ordinary way, as the other
// scans are.
#include "api.h"
#include "common.cuh"

namespace dlmk {
namespace {

__device__ __forceinline__ float sigmoid_g(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_g(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------------------------------------ gated scan
// Per head, S [dk, dv] in 32-bit:  S <- diag(a) S;  u = DELTA ? beta (v - S^T k) : v;  S <- S + k u^T;  o = S^T q.
// A block owns (head, request, a run of value columns).  Column j of S is shared by `parts` neighbouring lanes;
// lane `part` keeps rows part, part + parts, ... in registers.  S^T k and S^T q are added per lane and meet in a
// butterfly of shuffles, so the order of every sum is fixed by dk alone and a request's result does not depend on
// how its tokens were cut into steps.  Tokens are staged in tiles: a warp per token loads q and k, takes their
// lengths when they are to be unit vectors, and turns the raw decay and write strength into factors; then every
// thread walks the tile's tokens in order.
template <int NPT, bool DELTA>
__global__ void gated_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                                  const float* __restrict__ v, int ldv, const float* __restrict__ dec, int ldd,
                                  const float* __restrict__ beta, int ldb, const float* __restrict__ A_log,
                                  const float* __restrict__ dec_bias, float* state,
                                  const int32_t* __restrict__ cu_q, const int32_t* __restrict__ state_slot, float* o,
                                  int ldo, int heads, int qk_heads, int dk, int dv, int unit, float unit_eps,
                                  float q_scale, int decay_kind, float inv_tau, int parts, int tile) {
    dep_wait();
    extern __shared__ __align__(16) float sm[];           // [tile][3 dk + cols + 1]: q, k, a, v, beta
    const int h = blockIdx.x, r = blockIdx.y;
    const int cols = blockDim.x / parts;
    const int part = threadIdx.x % parts, col = threadIdx.x / parts;
    const int j0 = blockIdx.z * cols;
    const int j = j0 + col;
    const bool live = j < dv;
    const int ncols = min(cols, dv - j0);
    const int rl = 3 * dk + cols + 1;
    const int hq = h / (heads / qk_heads);
    float* st = state + ((long long)state_slot[r] * heads + h) * dk * dv;
    float s[NPT];
#pragma unroll
    for (int ii = 0; ii < NPT; ++ii) {
        const int i = part + parts * ii;
        s[ii] = (live && i < dk) ? st[(long long)i * dv + j] : 0.f;
    }
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const float neg_rate = decay_kind == 0 ? -expf(A_log[h]) : 0.f;
    const float bias0 = (decay_kind == 0 && dec_bias != nullptr) ? dec_bias[h] : 0.f;
    for (int first = t0; first < t1; first += tile) {
        const int n = min(tile, t1 - first);
        __syncthreads();                                   // the walk before has left the buffer
        for (int tok = warp; tok < n; tok += nwarp) {
            const long long t = first + tok;
            float* row = sm + (size_t)tok * rl;
            const float* qsrc = q + t * ldq + hq * dk;
            const float* ksrc = k + t * ldk + hq * dk;
            float sq = 0.f, sk = 0.f;
            for (int i = lane; i < dk; i += 32) {
                const float qv = qsrc[i], kv = ksrc[i];
                row[i] = qv;
                row[dk + i] = kv;
                sq = fmaf(qv, qv, sq);
                sk = fmaf(kv, kv, sk);
            }
            float fq = q_scale, fk = 1.0f;
            if (unit) {
                sq = warp_sum(sq);
                sk = warp_sum(sk);
                fq = q_scale * (1.0f / sqrtf(sq + unit_eps));
                fk = 1.0f / sqrtf(sk + unit_eps);
            }
            for (int i = lane; i < dk; i += 32) {
                row[i] *= fq;
                row[dk + i] *= fk;
            }
            if (decay_kind == 0) {
                if (lane == 0) row[2 * dk] = expf(neg_rate * softplus_g(dec[t * ldd + h] + bias0));
            } else {
                const float* dsrc = dec + t * ldd + h * dk;
                for (int i = lane; i < dk; i += 32) row[2 * dk + i] = expf(-softplus_g(-dsrc[i]) * inv_tau);
            }
            const float* vsrc = v + t * ldv + h * dv + j0;
            for (int c = lane; c < ncols; c += 32) row[3 * dk + c] = vsrc[c];
            if (lane == 0) row[3 * dk + cols] = DELTA ? sigmoid_g(beta[t * ldb + h]) : 0.f;
        }
        __syncthreads();
        for (int tok = 0; tok < n; ++tok) {
            const float* row = sm + (size_t)tok * rl;
            const float a0 = row[2 * dk];
            float kk[NPT], ksum = 0.f;
#pragma unroll
            for (int ii = 0; ii < NPT; ++ii) {
                const int i = part + parts * ii;
                kk[ii] = 0.f;
                if (i < dk) {
                    s[ii] *= decay_kind == 0 ? a0 : row[2 * dk + i];
                    kk[ii] = row[dk + i];
                    if (DELTA) ksum = fmaf(kk[ii], s[ii], ksum);
                }
            }
            float u = live ? row[3 * dk + col] : 0.f;
            if (DELTA) {
                for (int x = parts >> 1; x > 0; x >>= 1) ksum += __shfl_xor_sync(0xffffffffu, ksum, x);
                u = row[3 * dk + cols] * (u - ksum);
            }
            float acc = 0.f;
#pragma unroll
            for (int ii = 0; ii < NPT; ++ii) {
                const int i = part + parts * ii;
                if (i < dk) {
                    s[ii] = fmaf(kk[ii], u, s[ii]);
                    acc = fmaf(row[i], s[ii], acc);
                }
            }
            for (int x = parts >> 1; x > 0; x >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, x);
            if (live && part == 0) o[(long long)(first + tok) * ldo + h * dv + j] = acc;
        }
    }
#pragma unroll
    for (int ii = 0; ii < NPT; ++ii) {
        const int i = part + parts * ii;
        if (live && i < dk) st[(long long)i * dv + j] = s[ii];
    }
}

// ------------------------------------------------------------------- per-head norms, rotation, paged write
// One block a token, a warp a head.  x <- (x / sqrt(mean x^2 + eps)) * w over the head's d entries (w shared by
// the heads; nullptr: no norm), then the first rot_dims entries are rotated by position * inv_freq[pair]; q goes
// to q_out, k and v to the token's slot of the paged caches, every head D wide with zeros beyond its own size.
template <typename T>
__global__ void head_norm_rope_write_kernel(const float* qkv, int ld, const int32_t* __restrict__ positions,
                                            const float* __restrict__ qn_w, const float* __restrict__ kn_w, float eps,
                                            const float* __restrict__ inv_freq, int rot_dims, int interleaved,
                                            const int32_t* __restrict__ slots, T* q_out, T* k_cache, T* v_cache,
                                            int nh, int nkv, int d, int dv, int D, int page_size, int total_pages,
                                            int* err) {
    dep_wait();
    dep_launch_next();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const float* row = qkv + (long long)t * ld;
    const float pos = (float)positions[t];
    const int half = rot_dims / 2;
    int slot = slots != nullptr ? slots[t] : -1;
    if (slot >= total_pages * page_size) {
        if (threadIdx.x == 0) *err = 2;
        slot = -1;
    }
    const long long page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
    for (int hh = warp; hh < nh + 2 * nkv; hh += nwarp) {
        if (hh >= nh + nkv) {                               // a value head: copied as it is
            if (slot < 0) continue;
            const int g = hh - nh - nkv;
            const float* src = row + (long long)(nh + nkv) * d + (long long)g * dv;
            T* dst = v_cache + ((page * nkv + g) * page_size + off) * D;
            for (int i = lane; i < D; i += 32) dst[i] = from_f32<T>(i < dv ? src[i] : 0.f);
            continue;
        }
        const bool is_q = hh < nh;
        if (!is_q && slot < 0) continue;
        const float* src = row + (long long)hh * d;        // q heads, then k heads, all d wide
        const float* w = is_q ? qn_w : kn_w;
        float inv = 1.0f;
        if (w != nullptr) {
            float ss = 0.f;
            for (int i = lane; i < d; i += 32) ss = fmaf(src[i], src[i], ss);
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)d + eps);
        }
        T* dst = is_q ? q_out + ((long long)t * nh + hh) * D
                      : k_cache + ((page * nkv + (hh - nh)) * page_size + off) * D;
        for (int i = lane; i < D; i += 32) {
            float val = 0.f;
            if (i < d) {
                const float x = w != nullptr ? (src[i] * inv) * w[i] : src[i];
                val = x;
                if (i < 2 * half) {
                    int pi, f;
                    float sign;
                    if (interleaved) {
                        pi = i ^ 1; f = i >> 1; sign = (i & 1) ? 1.f : -1.f;
                    } else {
                        pi = i < half ? i + half : i - half; f = i < half ? i : i - half; sign = i < half ? -1.f : 1.f;
                    }
                    const float y = w != nullptr ? (src[pi] * inv) * w[pi] : src[pi];
                    float sn, cs;
                    sincosf(pos * inv_freq[f], &sn, &cs);
                    val = x * cs + sign * (y * sn);
                }
            }
            dst[i] = from_f32<T>(val);
        }
    }
}

// o[t, h * D + i] *= factor * sigmoid(gate[t * ldg + h]), in place
template <typename T>
__global__ void head_gate_kernel(T* o, const float* gate, int ldg, int nh, int D, float factor) {
    dep_wait();
    dep_launch_next();
    const int t = blockIdx.x;
    T* row = o + (long long)t * nh * D;
    for (int idx = threadIdx.x; idx < nh * D; idx += blockDim.x) {
        const float g = factor * sigmoid_g(gate[(long long)t * ldg + idx / D]);
        row[idx] = from_f32<T>(to_f32(row[idx]) * g);
    }
}

// resid[t] += (y[t] / rms(y[t])) * w_post;  then, with w_next, out[t] = (resid[t] / rms(resid[t])) * w_next
template <typename T>
__global__ void norm_add_norm_kernel(float* resid, const float* y, const float* __restrict__ w_post,
                                     const float* __restrict__ w_next, float eps, T* out, int H) {
    dep_wait();
    dep_launch_next();
    __shared__ float s_part[32];
    const int t = blockIdx.x;
    const float* yr = y + (long long)t * H;
    float* xr = resid + (long long)t * H;
    float part = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) part = fmaf(yr[i], yr[i], part);
    const float inv = 1.0f / sqrtf(block_sum(part, s_part) / (float)H + eps);
    part = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float x = xr[i] + (yr[i] * inv) * w_post[i];
        xr[i] = x;
        part = fmaf(x, x, part);
    }
    if (w_next == nullptr) return;
    const float inv2 = 1.0f / sqrtf(block_sum(part, s_part) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[(long long)t * H + i] = from_f32<T>((xr[i] * inv2) * w_next[i]);
}

// x[t] += (x0 != nullptr ? x0[t] : 0) + vec
__global__ void add_vec_rows_kernel(float* x, const float* x0, const float* __restrict__ vec, int H) {
    dep_wait();
    dep_launch_next();
    const long long base = (long long)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float a = x[base + i];
        if (x0 != nullptr) a += x0[base + i];
        x[base + i] = a + vec[i];
    }
}

}  // namespace

void gated_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* dec, int ldd,
                const float* beta, int ldb, const float* A_log, const float* dec_bias, float* state,
                const int32_t* cu_q, const int32_t* state_slot, float* o, int ldo, int R, int heads, int qk_heads,
                int dk, int dv, int unit, float unit_eps, float q_scale, int decay_kind, float tau,
                cudaStream_t stream) {
    if (R <= 0) return;
    DLM_CHECK(dk >= 1 && dk <= 512 && dv >= 1, "gated_scan: key size 1..512");
    DLM_CHECK(qk_heads >= 1 && heads % qk_heads == 0, "gated_scan: heads must be a multiple of the query/key heads");
    DLM_CHECK(decay_kind == 0 || decay_kind == 1, "gated_scan: decay kind 0 (per head) or 1 (per key channel)");
    DLM_CHECK(decay_kind == 1 || A_log != nullptr, "gated_scan: a decay per head needs its rates");
    DLM_CHECK(decay_kind == 0 || tau > 0.f, "gated_scan: tau must be positive");
    int parts = 1;
    const int want = dk > 64 ? 8 : 4;                        // rows a lane: short chains for small heads
    while (parts < 32 && (dk + parts - 1) / parts > want) parts *= 2;
    const int per = (dk + parts - 1) / parts;
    int cols = (parts >= 16 ? 256 : 128) / parts;
    while (cols > 1 && cols / 2 >= dv) cols /= 2;           // no more columns than the head has (a power of two)
    if (cols * parts < 32) cols = 32 / parts;                // at least a warp
    const int chunks = (dv + cols - 1) / cols;
    const int rl = 3 * dk + cols + 1;
    int tile = (40 * 1024) / (rl * (int)sizeof(float));
    tile = tile < 1 ? 1 : (tile > 32 ? 32 : tile);
    const size_t smem = (size_t)tile * rl * sizeof(float);
    const dim3 grid(heads, R, chunks);
    const float inv_tau = decay_kind == 1 ? 1.0f / tau : 0.f;
#define DLM_GSCAN(NPT, DELTA)                                                                                       \
    gated_scan_kernel<NPT, DELTA><<<grid, cols * parts, smem, stream>>>(q, ldq, k, ldk, v, ldv, dec, ldd, beta, ldb,  \
        A_log, dec_bias, state, cu_q, state_slot, o, ldo, heads, qk_heads, dk, dv, unit, unit_eps, q_scale,         \
        decay_kind, inv_tau, parts, tile)
    if (beta != nullptr) {
        if (per <= 4) DLM_GSCAN(4, true);
        else if (per <= 8) DLM_GSCAN(8, true);
        else DLM_GSCAN(16, true);
    } else {
        if (per <= 4) DLM_GSCAN(4, false);
        else if (per <= 8) DLM_GSCAN(8, false);
        else DLM_GSCAN(16, false);
    }
#undef DLM_GSCAN
    check_launch("gated_scan");
}

void head_norm_rope_write(const float* qkv, int ld, const int32_t* positions, const float* qn_w, const float* kn_w,
                          float eps, const float* inv_freq, int rot_dims, int interleaved, const int32_t* slots,
                          void* q_out, void* k_cache, void* v_cache, int T, int nh, int nkv, int d, int dv, int D,
                          int page_size, int total_pages, int dtype, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(D >= d && D >= dv, "head_norm_rope_write: the stored head size must hold keys and values");
    DLM_CHECK(rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= d, "head_norm_rope_write: rotated dims must be even and <= d");
    DLM_CHECK(rot_dims == 0 || inv_freq != nullptr, "head_norm_rope_write: a rotation needs its table");
    int* err = error_flag_ptr();
    if (dtype == F32)
        launch_dep(head_norm_rope_write_kernel<float>, dim3(T), dim3(128), 0, stream, qkv, ld, positions, qn_w, kn_w, eps,
                   inv_freq, rot_dims, interleaved, slots, static_cast<float*>(q_out), static_cast<float*>(k_cache),
                   static_cast<float*>(v_cache), nh, nkv, d, dv, D, page_size, total_pages, err);
    else
        launch_dep(head_norm_rope_write_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, qkv, ld, positions, qn_w,
                   kn_w, eps, inv_freq, rot_dims, interleaved, slots, static_cast<__nv_bfloat16*>(q_out),
                   static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), nh, nkv, d, dv, D,
                   page_size, total_pages, err);
    check_launch("head_norm_rope_write");
}

void head_gate(void* o, const float* gate, int ldg, int T, int nh, int D, float factor, int dtype, cudaStream_t stream) {
    if (T <= 0) return;
    if (dtype == F32)
        launch_dep(head_gate_kernel<float>, dim3(T), dim3(256), 0, stream, static_cast<float*>(o), gate, ldg, nh, D, factor);
    else
        launch_dep(head_gate_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, static_cast<__nv_bfloat16*>(o), gate,
                   ldg, nh, D, factor);
    check_launch("head_gate");
}

void norm_add_norm(float* resid, const float* y, const float* w_post, const float* w_next, float eps, void* out, int T,
                   int H, int out_dtype, cudaStream_t stream) {
    if (T <= 0) return;
    if (out_dtype == F32)
        launch_dep(norm_add_norm_kernel<float>, dim3(T), dim3(256), 0, stream, resid, y, w_post, w_next, eps,
                   static_cast<float*>(out), H);
    else
        launch_dep(norm_add_norm_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, resid, y, w_post, w_next, eps,
                   static_cast<__nv_bfloat16*>(out), H);
    check_launch("norm_add_norm");
}

void add_vec_rows(float* x, const float* x0, const float* vec, int T, int H, cudaStream_t stream) {
    if (T <= 0) return;
    launch_dep(add_vec_rows_kernel, dim3(T), dim3(256), 0, stream, x, x0, vec, H);
    check_launch("add_vec_rows");
}

}  // namespace dlmk
