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
// One 32-bit word from global to shared memory without holding a register for it; the thread that issued the copy
// sees it after copy_async_wait_all(), the others after the block's next barrier.
__device__ __forceinline__ void copy_async4(float* smem_dst, const float* gmem_src) {
    const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copy_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ gated scan
// Per head, S [dk, dv] in 32-bit:  S <- diag(a) S;  u = DELTA ? beta (v - S^T k) : v;  S <- S + k u^T;  o = S^T q.
// A block owns (head, request, a run of value columns).  Column j of S is shared by PARTS neighbouring lanes; a
// lane keeps NG groups of four neighbouring rows in registers (group ig * PARTS + part), so that q, k and the decays
// of its rows come from shared memory as 128-bit loads.  Rows beyond dk (up to 4 NG PARTS) are zeros with a decay
// of one and change nothing.  S^T k and S^T q are added per lane and meet in a butterfly of shuffles (one for both
// with the delta rule, whose read-out is taken from the decayed state and completed by u (k . q)), so the order
// of every sum is fixed by dk alone and a request's result does not depend on how its tokens were cut into steps.
// Tokens are staged in tiles in two buffers: while every thread walks one tile's tokens in order, asynchronous
// copies bring the next tile's raw values; a warp per token then takes the lengths of q and k when they are to be
// unit vectors and turns the raw decay and write strength into factors.
// What the recurrence with exponential gates and a running maximum (decay_kind 2) needs beside the common arguments.
struct MaxGateArgs {
    const float* igate; int ldi;        // raw input gate [T, heads] (the raw forget gate comes as `dec`)
    const float* i_bias; const float* f_bias;   // [heads]
    float cap, den_eps;
    float* nstate;                      // [slots, heads, dk]: the normaliser n
    float* mstate;                      // [slots, heads, dv + 1]: the running maximum, a copy per column
    float* rden;                        // [T, heads]: 1 / (max(|n . q|, exp(-m)) + den_eps)
};

__device__ __forceinline__ float log_sigmoid_g(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// decay_kind 2 (never with DELTA): per head a log input gate i = cap tanh((raw_i + bias) / cap) and a log forget
// gate f = log sigmoid(cap tanh((raw_f + bias) / cap)); with the running maximum m (carried in the state):
// m' = max(f + m, i); S <- exp(f + m - m') S + exp(i - m') k v^T.  The normaliser n <- exp(f + m - m') n + exp(i - m') k
// is kept as one more column of S (index dv, its "value" a constant one) by the block that owns that column; it
// writes 1 / (max(|n . q|, exp(-m')) + den_eps) per token and head instead of an output.  The maxima of a tile are
// taken by one thread in token order between two barriers; every block of a head does the same and keeps a copy of
// m of its own (one per column it owns), so no block reads what another writes.
template <int NG, int PARTS, bool DELTA>
__global__ void gated_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                                  const float* __restrict__ v, int ldv, const float* __restrict__ dec, int ldd,
                                  const float* __restrict__ beta, int ldb, const float* __restrict__ A_log,
                                  const float* __restrict__ dec_bias, float* state,
                                  const int32_t* __restrict__ cu_q, const int32_t* __restrict__ state_slot, float* o,
                                  int ldo, int heads, int qk_heads, int dk, int dv, int unit, float unit_eps,
                                  float q_scale, int decay_kind, float inv_tau, int tile, MaxGateArgs mg) {
    dep_wait();
    constexpr int DKP = 4 * NG * PARTS;                   // rows as the block keeps them
    extern __shared__ __align__(16) float sm[];           // 2 x [tile][q: DKP | k: DKP | a: DKP (a decay per channel) | v | a0, beta, k . q, -]
    const int h = blockIdx.x, r = blockIdx.y;
    const int cols = blockDim.x / PARTS;
    const int colsp = (cols + 3) & ~3;
    const int part = threadIdx.x % PARTS, col = threadIdx.x / PARTS;
    const int j0 = blockIdx.z * cols;
    const int j = j0 + col;
    const bool max_gate = !DELTA && decay_kind == 2;
    const int dvx = max_gate ? dv + 1 : dv;               // with the normaliser as one more column
    const bool live = j < dvx;
    const bool is_norm = max_gate && j == dv;
    const int ncols = min(cols, dvx - j0);
    const int off_v = (decay_kind == 1 ? 3 : 2) * DKP, off_s = off_v + colsp;
    const int rl = off_s + 4;
    const int hq = h / (heads / qk_heads);
    const long long slot_head = (long long)state_slot[r] * heads + h;
    float* st = state + slot_head * dk * dv;
    float* nst = max_gate ? mg.nstate + slot_head * dk : nullptr;
    float s[4 * NG];
#pragma unroll
    for (int ig = 0; ig < NG; ++ig)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = 4 * (ig * PARTS + part) + e;
            s[4 * ig + e] = (live && i < dk) ? (is_norm ? nst[i] : st[(long long)i * dv + j]) : 0.f;
        }
    float m_run = (max_gate && threadIdx.x == 0) ? mg.mstate[slot_head * (dv + 1) + j0] : 0.f;
    const float bias_i = max_gate ? mg.i_bias[h] : 0.f, bias_f = max_gate ? mg.f_bias[h] : 0.f;
    const int t0 = cu_q[r], t1 = cu_q[r + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const float neg_rate = decay_kind == 0 ? -expf(A_log[h]) : 0.f;
    const float bias0 = (decay_kind == 0 && dec_bias != nullptr) ? dec_bias[h] : 0.f;
    // Copies of a tile's raw values into one of the two buffers, without waiting: a warp a token, a lane the same
    // entries that it finishes later, so that a lane waits for its own copies only.
    auto fetch = [&](int first, float* buf) {
        const int n = min(tile, t1 - first);
        for (int tok = warp; tok < n; tok += nwarp) {
            const long long t = first + tok;
            float* row = buf + (size_t)tok * rl;
            const float* qsrc = q + t * ldq + hq * dk;
            const float* ksrc = k + t * ldk + hq * dk;
#pragma unroll
            for (int i = lane; i < DKP; i += 32) {
                if (i < dk) {
                    copy_async4(row + i, qsrc + i);
                    copy_async4(row + DKP + i, ksrc + i);
                } else {
                    row[i] = 0.f;
                    row[DKP + i] = 0.f;
                }
            }
            const float* vsrc = v + t * ldv + h * dv + j0;
            for (int c = lane; c < ncols; c += 32) {
                if (j0 + c < dv) copy_async4(row + off_v + c, vsrc + c);
                else row[off_v + c] = 1.0f;                // the normaliser's column takes k itself
            }
            if (decay_kind != 1) {
                if (lane == 0) {
                    copy_async4(row + off_s, dec + t * ldd + h);
                    if (max_gate) copy_async4(row + off_s + 1, mg.igate + t * mg.ldi + h);
                }
            } else {
                const float* dsrc = dec + t * ldd + h * dk;
#pragma unroll
                for (int i = lane; i < DKP; i += 32)
                    if (i < dk) copy_async4(row + 2 * DKP + i, dsrc + i);
            }
            if (DELTA && lane == 1) copy_async4(row + off_s + 1, beta + t * ldb + h);
        }
        copy_async_commit();
    };
    float* const buf0 = sm;
    float* const buf1 = sm + (size_t)tile * rl;
    if (t0 < t1) fetch(t0, buf0);
    int which = 0;
    for (int first = t0; first < t1; first += tile, which ^= 1) {
        const int n = min(tile, t1 - first);
        float* const cur = which ? buf1 : buf0;
        copy_async_wait_all();
        if (max_gate) {
            // log gates of the tile's tokens (a warp a token: its lane 0 issued both copies), then the running
            // maxima in token order by one thread: slots of a row become [f, i, m', f + m - m']
            for (int tok = warp; tok < n; tok += nwarp) {
                float* row = cur + (size_t)tok * rl;
                if (lane == 0) {
                    row[off_s] = log_sigmoid_g(mg.cap * tanhf((row[off_s] + bias_f) / mg.cap));
                    row[off_s + 1] = mg.cap * tanhf((row[off_s + 1] + bias_i) / mg.cap);
                }
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int tok = 0; tok < n; ++tok) {
                    float* row = cur + (size_t)tok * rl;
                    const float carried = row[off_s] + m_run;
                    const float m_new = fmaxf(carried, row[off_s + 1]);
                    row[off_s + 2] = m_new;
                    row[off_s + 3] = carried - m_new;
                    m_run = m_new;
                }
            }
            __syncthreads();
        }
        for (int tok = warp; tok < n; tok += nwarp) {      // lengths, decays and write strengths of the tile
            float* row = cur + (size_t)tok * rl;
            float qv[DKP / 32 > 0 ? DKP / 32 : 1], kv[DKP / 32 > 0 ? DKP / 32 : 1];
            float sq = 0.f, sk = 0.f, skq = 0.f;
#pragma unroll
            for (int ii = 0; ii * 32 < DKP; ++ii) {
                const int i = lane + 32 * ii;
                qv[ii] = i < DKP ? row[i] : 0.f;
                kv[ii] = i < DKP ? row[DKP + i] : 0.f;
                sq = fmaf(qv[ii], qv[ii], sq);
                sk = fmaf(kv[ii], kv[ii], sk);
                skq = fmaf(qv[ii], kv[ii], skq);
            }
            float fq = q_scale, fk = 1.0f;
            if (max_gate) {
                fk = expf(row[off_s + 1] - row[off_s + 2]);               // the write strength exp(i - m') rides on k
                if (lane == 0) row[off_s] = expf(row[off_s + 3]);         // the decay exp(f + m - m')
            } else if (decay_kind == 0) {
                if (lane == 0) row[off_s] = expf(neg_rate * softplus_g(row[off_s] + bias0));
            } else {
#pragma unroll
                for (int i = lane; i < DKP; i += 32)
                    row[2 * DKP + i] = i < dk ? expf(-softplus_g(-row[2 * DKP + i]) * inv_tau) : 1.0f;
            }
            if (lane == 1 && !max_gate) row[off_s + 1] = DELTA ? sigmoid_g(row[off_s + 1]) : 0.f;
            if (unit) {
                sq = warp_sum(sq);
                sk = warp_sum(sk);
                fq = q_scale * (1.0f / sqrtf(sq + unit_eps));
                fk *= 1.0f / sqrtf(sk + unit_eps);
            }
            if (DELTA) {
                skq = warp_sum(skq);
                if (lane == 2) row[off_s + 2] = skq * (fq * fk);
            }
#pragma unroll
            for (int ii = 0; ii * 32 < DKP; ++ii) {
                const int i = lane + 32 * ii;
                if (i < DKP) {
                    row[i] = qv[ii] * fq;
                    row[DKP + i] = kv[ii] * fk;
                }
            }
        }
        __syncthreads();                                   // the tile is ready, and the walk before has left the other buffer
        if (first + tile < t1) fetch(first + tile, which ? buf0 : buf1);
        const float* const sm_cur = cur;
#pragma unroll 2
        for (int tok = 0; tok < n; ++tok) {
            const float* row = sm_cur + (size_t)tok * rl;
            const float4* q4 = reinterpret_cast<const float4*>(row);
            const float4* k4 = reinterpret_cast<const float4*>(row + DKP);
            const float4* a4 = reinterpret_cast<const float4*>(row + 2 * DKP);
            const float4 sc = *reinterpret_cast<const float4*>(row + off_s);      // decay of the head, write strength, k . q
            float4 kk[NG];
            float acc;
            if (DELTA) {
                // Both read-outs are taken from the decayed state, so that they meet in one butterfly:
                // S'^T q = (aS)^T q + u (k . q) with S' = aS + k u^T; k . q comes with the tile.
                float ksum = 0.f, qsum = 0.f;
#pragma unroll
                for (int ig = 0; ig < NG; ++ig) {
                    const int g = ig * PARTS + part;
                    kk[ig] = k4[g];
                    const float4 qq = q4[g];
                    if (decay_kind == 0) {
                        s[4 * ig] *= sc.x; s[4 * ig + 1] *= sc.x; s[4 * ig + 2] *= sc.x; s[4 * ig + 3] *= sc.x;
                    } else {
                        const float4 a = a4[g];
                        s[4 * ig] *= a.x; s[4 * ig + 1] *= a.y; s[4 * ig + 2] *= a.z; s[4 * ig + 3] *= a.w;
                    }
                    float p = kk[ig].x * s[4 * ig], r = qq.x * s[4 * ig];
                    p = fmaf(kk[ig].y, s[4 * ig + 1], p); r = fmaf(qq.y, s[4 * ig + 1], r);
                    p = fmaf(kk[ig].z, s[4 * ig + 2], p); r = fmaf(qq.z, s[4 * ig + 2], r);
                    p = fmaf(kk[ig].w, s[4 * ig + 3], p); r = fmaf(qq.w, s[4 * ig + 3], r);
                    ksum += p;
                    qsum += r;
                }
#pragma unroll
                for (int x = PARTS >> 1; x > 0; x >>= 1) {
                    ksum += __shfl_xor_sync(0xffffffffu, ksum, x);
                    qsum += __shfl_xor_sync(0xffffffffu, qsum, x);
                }
                const float u = sc.y * ((live ? row[off_v + col] : 0.f) - ksum);
                acc = fmaf(u, sc.z, qsum);
#pragma unroll
                for (int ig = 0; ig < NG; ++ig) {
                    s[4 * ig] = fmaf(kk[ig].x, u, s[4 * ig]);
                    s[4 * ig + 1] = fmaf(kk[ig].y, u, s[4 * ig + 1]);
                    s[4 * ig + 2] = fmaf(kk[ig].z, u, s[4 * ig + 2]);
                    s[4 * ig + 3] = fmaf(kk[ig].w, u, s[4 * ig + 3]);
                }
            } else {
                const float u = live ? row[off_v + col] : 0.f;
                acc = 0.f;
#pragma unroll
                for (int ig = 0; ig < NG; ++ig) {
                    const int g = ig * PARTS + part;
                    kk[ig] = k4[g];
                    const float4 qq = q4[g];
                    if (decay_kind != 1) {
                        s[4 * ig] *= sc.x; s[4 * ig + 1] *= sc.x; s[4 * ig + 2] *= sc.x; s[4 * ig + 3] *= sc.x;
                    } else {
                        const float4 a = a4[g];
                        s[4 * ig] *= a.x; s[4 * ig + 1] *= a.y; s[4 * ig + 2] *= a.z; s[4 * ig + 3] *= a.w;
                    }
                    s[4 * ig] = fmaf(kk[ig].x, u, s[4 * ig]);
                    s[4 * ig + 1] = fmaf(kk[ig].y, u, s[4 * ig + 1]);
                    s[4 * ig + 2] = fmaf(kk[ig].z, u, s[4 * ig + 2]);
                    s[4 * ig + 3] = fmaf(kk[ig].w, u, s[4 * ig + 3]);
                    float p = qq.x * s[4 * ig];
                    p = fmaf(qq.y, s[4 * ig + 1], p);
                    p = fmaf(qq.z, s[4 * ig + 2], p);
                    p = fmaf(qq.w, s[4 * ig + 3], p);
                    acc += p;
                }
#pragma unroll
                for (int x = PARTS >> 1; x > 0; x >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, x);
            }
            if (live && part == 0) {
                if (is_norm)
                    mg.rden[(long long)(first + tok) * heads + h] = 1.0f / (fmaxf(fabsf(acc), expf(-sc.z)) + mg.den_eps);
                else
                    o[(long long)(first + tok) * ldo + h * dv + j] = acc;
            }
        }
    }
#pragma unroll
    for (int ig = 0; ig < NG; ++ig)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = 4 * (ig * PARTS + part) + e;
            if (live && i < dk) {
                if (is_norm) nst[i] = s[4 * ig + e];
                else st[(long long)i * dv + j] = s[4 * ig + e];
            }
        }
    if (max_gate && threadIdx.x == 0)
        for (int c = 0; c < ncols; ++c) mg.mstate[slot_head * (dv + 1) + j0 + c] = m_run;
}

// ------------------------------------------------------------------- per-head norms, rotation, paged write
// A warp a head: block (t, y) takes heads y * warps .. of token t.  x <- (x / sqrt(mean x^2 + eps)) * w over the
// head's d entries (w shared by the heads; nullptr: no norm), kept in shared memory; then the first rot_dims entries
// are rotated by position * inv_freq[pair], a lane a pair; q goes to q_out, k and v to the token's slot of the
// paged caches, every head D wide with zeros beyond its own size.
template <typename T>
__global__ void head_norm_rope_write_kernel(const float* __restrict__ qkv, int ld, const int32_t* __restrict__ positions,
                                            const float* __restrict__ qn_w, const float* __restrict__ kn_w, float eps,
                                            const float* __restrict__ inv_freq, int rot_dims, int interleaved,
                                            const int32_t* __restrict__ slots, T* __restrict__ q_out,
                                            T* __restrict__ k_cache, T* __restrict__ v_cache, int nh, int nkv, int d,
                                            int dv, int D, int page_size, int total_pages,
                                            int* err) {
    dep_wait();
    dep_launch_next();
    extern __shared__ __align__(16) float head_stage[];    // [warps][d], [2][half]
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
    float* sincos = head_stage + nwarp * d;                // [2][half]: the token's sines and cosines, once a block
    for (int f = threadIdx.x; f < half; f += blockDim.x) sincosf(pos * inv_freq[f], sincos + f, sincos + half + f);
    __syncthreads();
    for (int hh = blockIdx.y * nwarp + warp; hh < nh + 2 * nkv; hh += gridDim.y * nwarp) {
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
        float* sh = head_stage + warp * d;                  // the head as it is after the norm
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float x = src[i];
            sh[i] = x;
            ss = fmaf(x, x, ss);
        }
        if (w != nullptr) {
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)d + eps);
            for (int i = lane; i < d; i += 32) sh[i] = (sh[i] * inv) * w[i];      // a lane rereads what it wrote
        }
        __syncwarp();
        T* dst = is_q ? q_out + ((long long)t * nh + hh) * D
                      : k_cache + ((page * nkv + (hh - nh)) * page_size + off) * D;
        for (int f = lane; f < half; f += 32) {             // a lane a pair
            const int ia = interleaved ? 2 * f : f, ib = interleaved ? 2 * f + 1 : f + half;
            const float x = sh[ia], y = sh[ib];
            const float sn = sincos[f], cs = sincos[half + f];
            dst[ia] = from_f32<T>(x * cs - y * sn);
            dst[ib] = from_f32<T>(y * cs + x * sn);
        }
        for (int i = 2 * half + lane; i < D; i += 32) dst[i] = from_f32<T>(i < d ? sh[i] : 0.f);
        __syncwarp();                                       // the next head takes the same staging row
    }
}

// o[t, h * D + i] *= factor * sigmoid(gate[t * ldg + h]), in place
template <typename T>
__global__ void head_gate_kernel(T* o, const float* gate, int ldg, int nh, int D, float factor) {
    dep_wait();
    dep_launch_next();
    const int t = blockIdx.x;
    T* row = o + (long long)t * nh * D;
    constexpr int U = 4;
    for (int i0 = threadIdx.x; i0 < nh * D; i0 += U * blockDim.x) {
        float g[U], v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = i0 + u * blockDim.x;
            g[u] = idx < nh * D ? gate[(long long)t * ldg + idx / D] : 0.f;
            v[u] = idx < nh * D ? to_f32(row[idx]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = i0 + u * blockDim.x;
            if (idx < nh * D) row[idx] = from_f32<T>(v[u] * (factor * sigmoid_g(g[u])));
        }
    }
}

// resid[t] += (y[t] / rms(y[t])) * w_post;  then, with w_next, out[t] = (resid[t] / rms(resid[t])) * w_next.
// `staged`: the two rows are read from global memory once, side by side, and kept in shared memory ([2][H]) for the
// later passes (a thread rereads only its own entries); otherwise the later passes read global memory again.
template <typename T>
__global__ void norm_add_norm_kernel(float* __restrict__ resid, const float* __restrict__ y,
                                     const float* __restrict__ w_post, const float* __restrict__ w_next, float eps,
                                     T* __restrict__ out, int H, int staged) {
    dep_wait();
    dep_launch_next();
    __shared__ float s_part[32];
    extern __shared__ __align__(16) float row_stage[];
    constexpr int U = 4;                                   // loads in flight a thread; the sums keep their order
    const int t = blockIdx.x, step = blockDim.x;
    const float* yr = y + (long long)t * H;
    float* xr = resid + (long long)t * H;
    const float* ys = staged ? row_stage : yr;
    float* xs = staged ? row_stage + H : xr;
    float part = 0.f;
    for (int i0 = threadIdx.x; i0 < H; i0 += U * step) {
        float yv[U], xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * step;
            yv[u] = i < H ? yr[i] : 0.f;
            xv[u] = (staged && i < H) ? xr[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * step;
            if (i < H) {
                if (staged) {
                    row_stage[i] = yv[u];
                    row_stage[H + i] = xv[u];
                }
                part = fmaf(yv[u], yv[u], part);
            }
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(part, s_part) / (float)H + eps);
    part = 0.f;
    for (int i0 = threadIdx.x; i0 < H; i0 += U * step) {
        float yv[U], xv[U], wv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * step;
            yv[u] = i < H ? ys[i] : 0.f;
            xv[u] = i < H ? xs[i] : 0.f;
            wv[u] = i < H ? w_post[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * step;
            if (i < H) {
                const float x = xv[u] + (yv[u] * inv) * wv[u];
                xs[i] = x;
                if (staged) xr[i] = x;
                part = fmaf(x, x, part);
            }
        }
    }
    if (w_next == nullptr) return;
    const float inv2 = 1.0f / sqrtf(block_sum(part, s_part) / (float)H + eps);
    for (int i0 = threadIdx.x; i0 < H; i0 += U * step) {
        float xv[U], wv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * step;
            xv[u] = i < H ? xs[i] : 0.f;
            wv[u] = i < H ? w_next[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * step;
            if (i < H) out[(long long)t * H + i] = from_f32<T>((xv[u] * inv2) * wv[u]);
        }
    }
}

// x[t] += (x0 != nullptr ? x0[t] : 0) + vec
__global__ void add_vec_rows_kernel(float* x, const float* x0, const float* __restrict__ vec, int H) {
    dep_wait();
    dep_launch_next();
    const long long base = (long long)blockIdx.x * H;
    constexpr int U = 4;
    for (int i0 = threadIdx.x; i0 < H; i0 += U * blockDim.x) {
        float a[U], b[U], c[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * blockDim.x;
            a[u] = i < H ? x[base + i] : 0.f;
            b[u] = (x0 != nullptr && i < H) ? x0[base + i] : 0.f;
            c[u] = i < H ? vec[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = i0 + u * blockDim.x;
            if (i < H) x[base + i] = (x0 != nullptr ? a[u] + b[u] : a[u]) + c[u];
        }
    }
}

}  // namespace

namespace {

void launch_gated_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* dec,
                       int ldd, const float* beta, int ldb, const float* A_log, const float* dec_bias, float* state,
                       const int32_t* cu_q, const int32_t* state_slot, float* o, int ldo, int R, int heads,
                       int qk_heads, int dk, int dv_own, int unit, float unit_eps, float q_scale, int decay_kind,
                       float tau, MaxGateArgs mg, cudaStream_t stream) {
    const int dv = decay_kind == 2 ? dv_own + 1 : dv_own;    // columns the blocks share out (the normaliser is one)
    // rows a lane keeps: 4 NG, over PARTS lanes a column (short chains for small heads)
    const int ng = dk <= 64 ? 1 : (dk <= 256 ? 2 : 4);
    const int parts = dk <= 16 ? 4 : (dk <= 32 ? 8 : (dk <= 128 ? 16 : 32));
    const int dkp = 4 * ng * parts;
    int cols = (parts >= 16 ? 256 : 128) / parts;
    while (cols > 1 && cols / 2 >= dv) cols /= 2;           // no more columns than the head has (a power of two)
    if (cols * parts < 32) cols = 32 / parts;                // at least a warp
    const int chunks = (dv + cols - 1) / cols;
    const int rl = (decay_kind == 1 ? 3 : 2) * dkp + ((cols + 3) & ~3) + 4;
    int tile = (23 * 1024) / (rl * (int)sizeof(float));     // two buffers within 48 KB
    tile = tile < 1 ? 1 : (tile > 32 ? 32 : tile);
    const size_t smem = (size_t)2 * tile * rl * sizeof(float);
    const dim3 grid(heads, R, chunks);
    const float inv_tau = decay_kind == 1 ? 1.0f / tau : 0.f;
#define DLM_GSCAN(NG, PARTS, DELTA)                                                                                 \
    gated_scan_kernel<NG, PARTS, DELTA><<<grid, cols * parts, smem, stream>>>(q, ldq, k, ldk, v, ldv, dec, ldd,     \
        beta, ldb, A_log, dec_bias, state, cu_q, state_slot, o, ldo, heads, qk_heads, dk, dv_own, unit, unit_eps,   \
        q_scale, decay_kind, inv_tau, tile, mg)
#define DLM_GSCAN_SIZES(DELTA)                                                                                      \
    do {                                                                                                            \
        if (dkp == 16) DLM_GSCAN(1, 4, DELTA);                                                                      \
        else if (dkp == 32) DLM_GSCAN(1, 8, DELTA);                                                                 \
        else if (dkp == 64) DLM_GSCAN(1, 16, DELTA);                                                                \
        else if (dkp == 128) DLM_GSCAN(2, 16, DELTA);                                                               \
        else if (dkp == 256) DLM_GSCAN(2, 32, DELTA);                                                               \
        else DLM_GSCAN(4, 32, DELTA);                                                                               \
    } while (0)
    if (beta != nullptr) DLM_GSCAN_SIZES(true);
    else DLM_GSCAN_SIZES(false);
#undef DLM_GSCAN_SIZES
#undef DLM_GSCAN
    check_launch("gated_scan");
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
    launch_gated_scan(q, ldq, k, ldk, v, ldv, dec, ldd, beta, ldb, A_log, dec_bias, state, cu_q, state_slot, o, ldo, R,
                      heads, qk_heads, dk, dv, unit, unit_eps, q_scale, decay_kind, tau, MaxGateArgs{}, stream);
}

void memory_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* igate, int ldi,
                 const float* fgate, int ldf, const float* i_bias, const float* f_bias, float cap, float* state,
                 float* nstate, float* mstate, const int32_t* cu_q, const int32_t* state_slot, float* o, int ldo,
                 float* rden, int R, int heads, int dk, int dv, float q_scale, float den_eps, cudaStream_t stream) {
    if (R <= 0) return;
    DLM_CHECK(dk >= 1 && dk <= 512 && dv >= 1, "memory_scan: key size 1..512");
    DLM_CHECK(cap > 0.f, "memory_scan: the gates' cap must be positive");
    DLM_CHECK(i_bias != nullptr && f_bias != nullptr && nstate != nullptr && mstate != nullptr && rden != nullptr,
              "memory_scan: gate biases, normaliser, maximum and the denominators' place are needed");
    const MaxGateArgs mg{igate, ldi, i_bias, f_bias, cap, den_eps, nstate, mstate, rden};
    launch_gated_scan(q, ldq, k, ldk, v, ldv, fgate, ldf, nullptr, 0, nullptr, nullptr, state, cu_q, state_slot, o, ldo,
                      R, heads, heads, dk, dv, 0, 0.f, q_scale, 2, 0.f, mg, stream);
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
    const int warps = 8;
    int gy = (nh + 2 * nkv + warps - 1) / warps;            // a head a warp while the blocks are few (a decode step);
    while (gy > 1 && (long long)T * gy > 16 * 148) gy = (gy + 1) / 2;   // on a prompt several heads a warp: a block's
    const dim3 grid(T, gy);                                  // opening (slot, sines) is most of a one-head warp's work
    const size_t stage = ((size_t)warps * d + rot_dims) * sizeof(float);
    DLM_CHECK(stage <= 48 * 1024, "head_norm_rope_write: head size too large");
    if (dtype == F32)
        launch_dep(head_norm_rope_write_kernel<float>, grid, dim3(32 * warps), stage, stream, qkv, ld, positions, qn_w, kn_w, eps,
                   inv_freq, rot_dims, interleaved, slots, static_cast<float*>(q_out), static_cast<float*>(k_cache),
                   static_cast<float*>(v_cache), nh, nkv, d, dv, D, page_size, total_pages, err);
    else
        launch_dep(head_norm_rope_write_kernel<__nv_bfloat16>, grid, dim3(32 * warps), stage, stream, qkv, ld, positions, qn_w,
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
    const size_t rows = (size_t)2 * H * sizeof(float);
    const int staged = rows <= 40 * 1024 ? 1 : 0;
    const size_t smem = staged ? rows : 0;
    const dim3 block(H > 2048 ? 512 : 256);
    if (out_dtype == F32)
        launch_dep(norm_add_norm_kernel<float>, dim3(T), block, smem, stream, resid, y, w_post, w_next, eps,
                   static_cast<float*>(out), H, staged);
    else
        launch_dep(norm_add_norm_kernel<__nv_bfloat16>, dim3(T), block, smem, stream, resid, y, w_post, w_next, eps,
                   static_cast<__nv_bfloat16*>(out), H, staged);
    check_launch("norm_add_norm");
}

void add_vec_rows(float* x, const float* x0, const float* vec, int T, int H, cudaStream_t stream) {
    if (T <= 0) return;
    launch_dep(add_vec_rows_kernel, dim3(T), dim3(256), 0, stream, x, x0, vec, H);
    check_launch("add_vec_rows");
}

}  // namespace dlmk
