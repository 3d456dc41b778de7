// Attention through a cached latent: per token the cache holds one normalised latent vector c (`rank` wide)
// and one rotated key part (`dr` wide) shared by all heads; keys and values of a head are W_uk c and W_uv c.
// The kernels never build them: a head's query is taken through W_uk once (q' = W_uk^T q, `rank` wide), scores
// are q' . c + q_rot . k_rot, the weighted sum of the latents goes through W_uv at the end.  Sliding window,
// a sink in the softmax's denominator (a learned logit per head without key or value), a gate on each head's
// output.  Scores, softmax and every sum are 32-bit.
//
// The two per-head products (queries through W_uk, weighted latents through W_uv) are grouped matrix products
// with the heads as groups, outside this file; the kernels here split and rotate the queries, attend over the
// latent rows, and gate the values.  The latent rows are shared by all heads, so a block serves a token and up to
// eight of its heads and reads each row once.  In 32-bit a (token, head)'s result is computed in one order whatever else the step holds (keys
// go in chunks cut at absolute positions, one after the other); in bfloat16 a step of few tokens cuts each token's
// keys over several blocks and merges them, which changes the result by rounding only.
#include <cstdlib>

#include "api.h"
#include "common.cuh"
#include "mma_sync.cuh"

namespace dlmk {
namespace {

// Per token: c_q = rmsnorm(proj[off_q : off_q + q_rank]) * qn_w  -> cq_out (activation dtype, feeds a product);
// c = rmsnorm(proj[off_kv : off_kv + rank]) * kvn_w and k_rot = rotate(proj[off_kv + rank : + dr]) -> the cache row
// of the token's slot, [rank | dr].  Rotation: entry i < rot_dims / 2 pairs with i + rot_dims / 2, angle
// position * inv_freq[i] in 32-bit; entries from rot_dims on pass unchanged.
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ proj, int ld, int off_q, int q_rank,
                                   const float* __restrict__ qn_w, int off_kv, int rank, const float* __restrict__ kvn_w,
                                   int dr, const float* __restrict__ inv_freq, int rot_dims, int interleaved,
                                   const int32_t* __restrict__ positions, const int32_t* __restrict__ slots, float eps,
                                   T* cq_out, T* cache, int page_size, int total_pages, int* err) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    __shared__ float s_part[32];
    const int t = blockIdx.x;
    const float* row = proj + (long long)t * ld;
    // the query latent
    if (q_rank > 0) {
        float part = 0.f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) part = fmaf(row[off_q + i], row[off_q + i], part);
        const float ss = block_sum(part, s_part);
        const float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            cq_out[(long long)t * q_rank + i] = from_f32<T>((row[off_q + i] * inv) * qn_w[i]);
    }
    if (slots == nullptr) return;
    const int s = slots[t];
    if (s < 0) return;
    if (s >= total_pages * page_size) {
        if (threadIdx.x == 0) *err = 2;
        return;
    }
    T* dst = cache + (long long)s * (rank + dr);
    float part = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) part = fmaf(row[off_kv + i], row[off_kv + i], part);
    const float ss = block_sum(part, s_part);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<T>((row[off_kv + i] * inv) * kvn_w[i]);
    const float* kr = row + off_kv + rank;
    const int half = rot_dims / 2;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < dr; i += blockDim.x) {
        float v;
        if (interleaved && i < 2 * half) {
            float sn, cs;
            sincosf(pos * inv_freq[i >> 1], &sn, &cs);
            v = (i & 1) ? kr[i] * cs + kr[i - 1] * sn : kr[i] * cs - kr[i + 1] * sn;
        } else if (i < half) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            v = kr[i] * cs - kr[i + half] * sn;
        } else if (i < 2 * half) {
            float sn, cs;
            sincosf(pos * inv_freq[i - half], &sn, &cs);
            v = kr[i] * cs + kr[i - half] * sn;
        } else {
            v = kr[i];
        }
        dst[rank + i] = from_f32<T>(v);
    }
}

constexpr int LA_THREADS = 256;   // 8 warps
constexpr int LA_KC = 32;         // keys a chunk: one per lane where a warp takes the softmax of a chunk
constexpr int LA_HG = 8;          // most heads a block serves: the latent rows it stages are shared by all of them

template <typename T> struct Vec16;       // how many elements a 16-byte load brings
template <> struct Vec16<float> { static constexpr int n = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int n = 8; };

// Splits the projected queries q[T, H * (dn + dr)] (per head [dn plain | dr to be rotated]): the plain parts go
// head by head to qn[H, T, dn] in the activation dtype (the left operand of the per-head product with W_uk), the
// rotated parts, rotated, to qr[T, H, dr] in 32-bit.
template <typename T>
__global__ void latent_q_split_kernel(const float* __restrict__ q, int ldq, const int32_t* __restrict__ positions,
                                      const float* __restrict__ inv_freq, int rot_dims, int interleaved, T* qn,
                                      float* qr, int Tn, int H, int dn, int dr) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    const int t = blockIdx.x;
    const int half = rot_dims / 2;
    const float pos = (float)positions[t];
    for (int idx = threadIdx.x; idx < H * (dn + dr); idx += blockDim.x) {
        const int h = idx / (dn + dr), i = idx - h * (dn + dr);
        const float* row = q + (long long)t * ldq + (long long)h * (dn + dr);
        if (i < dn) {
            qn[((long long)h * Tn + t) * dn + i] = from_f32<T>(row[i]);
            continue;
        }
        const float* r = row + dn;
        const int e = i - dn;
        float v;
        if (interleaved && e < 2 * half) {
            float sn, cs;
            sincosf(pos * inv_freq[e >> 1], &sn, &cs);
            v = (e & 1) ? r[e] * cs + r[e - 1] * sn : r[e] * cs - r[e + 1] * sn;
        } else if (e < half) {
            float sn, cs;
            sincosf(pos * inv_freq[e], &sn, &cs);
            v = r[e] * cs - r[e + half] * sn;
        } else if (e < 2 * half) {
            float sn, cs;
            sincosf(pos * inv_freq[e - half], &sn, &cs);
            v = r[e] * cs + r[e - half] * sn;
        } else {
            v = r[e];
        }
        qr[((long long)t * H + h) * dr + e] = v;
    }
}

// out[t, h * dv + d] = val[h * T + t, d] * sigmoid(gate[t, h])  (gate == nullptr: 1): the per-head values back
// token by token, gated, in the activation dtype.
template <typename T>
__global__ void latent_gate_out_kernel(const float* __restrict__ val, const float* __restrict__ gate, int ldg, T* out,
                                       int Tn, int H, int dv) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    const int t = blockIdx.x;
    for (int idx = threadIdx.x; idx < H * dv; idx += blockDim.x) {
        const int h = idx / dv, d = idx - h * dv;
        const float g = gate ? 1.0f / (1.0f + expf(-gate[(long long)t * ldg + h])) : 1.0f;
        out[(long long)t * H * dv + idx] = from_f32<T>(val[((long long)h * Tn + t) * dv + d] * g);
    }
}

// One block a (token, group of up to LA_HG heads, split of the token's keys).  q_lat[H, T, rank] holds the heads'
// queries already taken through W_uk, q_rot[T, H, dr] their rotated parts.  The block walks its chunks of LA_KC
// keys (chunks are cut at absolute multiples of LA_KC, so a token's sums have one order whatever else the step
// holds): the chunk's cache rows are staged in shared memory, every warp scores four of them against all heads,
// warp g takes head g's softmax step over the chunk (running maximum, sum, rescale), and every thread adds the
// chunk's rows into its columns of every head's weighted latent.  NCOL: columns of the latent a thread owns
// (rank <= 256 NCOL).  With one split the block normalises (the sink joins the maximum and the denominator) and
// stores lat[H, T, rank]; with more it leaves (maximum, sum, weighted latent) per head for the merge kernel.
template <typename T, int NCOL>
__global__ void __launch_bounds__(LA_THREADS)
latent_attention_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot, const float* __restrict__ sink,
                        const T* __restrict__ cache, const int32_t* __restrict__ block_table, int table_width,
                        const int32_t* __restrict__ token_req, const int32_t* __restrict__ positions, T* lat,
                        float* partial, int Tn, int H, int dr, int rank, int page_size, int total_pages, int window,
                        float scale, int hg_max, int n_splits, int* err) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    // (a long kernel, launched in the ordinary way: its blocks are placed when the machine is free, and the
    // kernel after it is let in only when it ends)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int width = rank + dr;
    const int wpad = (width + 7) & ~7;                      // row pitch of the staged keys (16-byte multiples)
    float* s_qa = reinterpret_cast<float*>(smem_raw);       // [LA_HG][rank]  queries through W_uk
    float* s_qr = s_qa + (size_t)LA_HG * rank;              // [LA_HG][dr]    rotated query parts
    float* s_p = s_qr + (size_t)LA_HG * dr;                 // [LA_HG][LA_KC] scores, then weights, of a chunk
    float* s_m = s_p + LA_HG * LA_KC;                       // [LA_HG] running maximum
    float* s_l = s_m + LA_HG;                               // [LA_HG] running sum
    float* s_corr = s_l + LA_HG;                            // [LA_HG] rescale of this chunk
    T* s_keys = reinterpret_cast<T*>(s_corr + LA_HG);       // [LA_KC][wpad]
    const int t = blockIdx.x;
    const int h0 = blockIdx.y * hg_max;
    const int hg = min(hg_max, H - h0);
    const int ks = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = positions[t];
    for (int idx = threadIdx.x; idx < hg * rank; idx += LA_THREADS) {
        const int g = idx / rank, r = idx - g * rank;
        s_qa[idx] = q_lat[((long long)(h0 + g) * Tn + t) * rank + r];
    }
    for (int idx = threadIdx.x; idx < hg * dr; idx += LA_THREADS) s_qr[idx] = q_rot[((long long)t * H + h0) * dr + idx];
    if (threadIdx.x < LA_HG) {
        s_m[threadIdx.x] = -INFINITY;
        s_l[threadIdx.x] = 0.f;
    }
    float acc[LA_HG][NCOL];
#pragma unroll
    for (int g = 0; g < LA_HG; ++g)
#pragma unroll
        for (int c = 0; c < NCOL; ++c) acc[g][c] = 0.f;

    const int req = token_req[t];
    const int32_t* table = block_table + (long long)req * table_width;
    const int lo = window > 0 ? max(p - window + 1, 0) : 0;
    const int c_first = lo / LA_KC, c_last = p / LA_KC;
    const int per = (c_last - c_first + 1 + n_splits - 1) / n_splits;
    const int c_begin = c_first + ks * per, c_end = min(c_begin + per, c_last + 1);
    const bool vec = (width % Vec16<T>::n) == 0;
    for (int ch = c_begin; ch < c_end; ++ch) {
        __syncthreads();                                    // the chunk before is done with s_keys and s_p
        // ---- stage the chunk's rows (zeros where the token sees no key)
        for (int jj = warp; jj < LA_KC; jj += LA_THREADS / 32) {
            const int j = ch * LA_KC + jj;
            T* dst = s_keys + (size_t)jj * wpad;
            const T* row = nullptr;
            if (j >= lo && j <= p) {
                const int lp = j / page_size;
                const int page = lp < table_width ? table[lp] : -1;
                if (page < 0 || page >= total_pages) {
                    if (lane == 0) *err = 3;
                } else {
                    row = cache + ((long long)page * page_size + (j - lp * page_size)) * width;
                }
            }
            if (row == nullptr) {
                for (int i = lane; i < wpad; i += 32) dst[i] = from_f32<T>(0.f);
            } else if (vec) {
                const uint4* src = reinterpret_cast<const uint4*>(row);
                uint4* d4 = reinterpret_cast<uint4*>(dst);
                for (int i = lane; i < width / Vec16<T>::n; i += 32) d4[i] = src[i];
            } else {
                for (int i = lane; i < width; i += 32) dst[i] = row[i];
            }
        }
        __syncthreads();
        // ---- scores of this warp's four keys against every head
        for (int jj = warp; jj < LA_KC; jj += LA_THREADS / 32) {
            const int j = ch * LA_KC + jj;
            const T* row = s_keys + (size_t)jj * wpad;
            float kreg[8 * NCOL];
#pragma unroll
            for (int n = 0; n < 8 * NCOL; ++n) {
                const int r = lane + 32 * n;
                kreg[n] = r < rank ? to_f32(row[r]) : 0.f;
            }
            for (int g = 0; g < hg; ++g) {
                const float* qa = s_qa + (size_t)g * rank;
                float dot = 0.f;
#pragma unroll
                for (int n = 0; n < 8 * NCOL; ++n) {
                    const int r = lane + 32 * n;
                    if (r < rank) dot = fmaf(qa[r], kreg[n], dot);
                }
                for (int i = lane; i < dr; i += 32) dot = fmaf(s_qr[g * dr + i], to_f32(row[rank + i]), dot);
                dot = warp_sum(dot);
                if (lane == 0) s_p[g * LA_KC + jj] = (j >= lo && j <= p) ? dot * scale : -INFINITY;
            }
        }
        __syncthreads();
        // ---- head g's softmax step over the chunk, by warp g
        if (warp < hg) {
            const float sc = s_p[warp * LA_KC + lane];
            const float m_old = s_m[warp];
            const float m_new = fmaxf(m_old, warp_max(sc));
            float pw = 0.f, corr = 1.f;
            if (m_new > -INFINITY) {
                pw = expf(sc - m_new);                      // a key the token does not see: exp(-inf) = 0
                corr = expf(m_old - m_new);                 // nothing before this chunk: exp(-inf) = 0
            }
            const float sum = warp_sum(pw);
            s_p[warp * LA_KC + lane] = pw;
            if (lane == 0) {
                s_l[warp] = s_l[warp] * corr + sum;
                s_m[warp] = m_new;
                s_corr[warp] = corr;
            }
        }
        __syncthreads();
        // ---- weighted latents: every thread its columns, all heads
#pragma unroll
        for (int c = 0; c < NCOL; ++c) {
            const int r = threadIdx.x + LA_THREADS * c;
            if (r < rank) {
#pragma unroll
                for (int g = 0; g < LA_HG; ++g)
                    if (g < hg) acc[g][c] *= s_corr[g];
                for (int jj = 0; jj < LA_KC; jj += 4) {
                    const float k0 = to_f32(s_keys[(size_t)(jj + 0) * wpad + r]), k1 = to_f32(s_keys[(size_t)(jj + 1) * wpad + r]);
                    const float k2 = to_f32(s_keys[(size_t)(jj + 2) * wpad + r]), k3 = to_f32(s_keys[(size_t)(jj + 3) * wpad + r]);
#pragma unroll
                    for (int g = 0; g < LA_HG; ++g) {
                        if (g < hg) {
                            const float4 pw = *reinterpret_cast<const float4*>(s_p + g * LA_KC + jj);
                            float a = acc[g][c];
                            a = fmaf(pw.x, k0, a);
                            a = fmaf(pw.y, k1, a);
                            a = fmaf(pw.z, k2, a);
                            a = fmaf(pw.w, k3, a);
                            acc[g][c] = a;
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < LA_HG; ++g) {
        if (g < hg) {
            if (n_splits > 1) {
                // (maximum, sum, weighted latent) of this split
                float* dst = partial + (((long long)t * H + h0 + g) * n_splits + ks) * (rank + 2);
                if (threadIdx.x == 0) {
                    dst[0] = s_m[g];
                    dst[1] = s_l[g];
                }
#pragma unroll
                for (int c = 0; c < NCOL; ++c) {
                    const int r = threadIdx.x + LA_THREADS * c;
                    if (r < rank) dst[2 + r] = acc[g][c];
                }
            } else {
                // normalise with the sink in the maximum and the denominator
                const float snk = sink ? sink[h0 + g] : -INFINITY;
                const float mm = fmaxf(s_m[g], snk);
                const float f = s_l[g] > 0.f ? expf(s_m[g] - mm) : 0.f;
                const float den = s_l[g] * f + (sink ? expf(snk - mm) : 0.f);
                const float w = den > 0.f ? f / den : 0.f;
                T* dst = lat + ((long long)(h0 + g) * Tn + t) * rank;
#pragma unroll
                for (int c = 0; c < NCOL; ++c) {
                    const int r = threadIdx.x + LA_THREADS * c;
                    if (r < rank) dst[r] = from_f32<T>(acc[g][c] * w);
                }
            }
        }
    }
}

// The same on tensor cores (bfloat16, latent size a multiple of 128 up to 512): one block a (token, up to 16 heads,
// split).  The heads are the 16 rows of m16n8k16 products.  Per chunk of 32 keys: scores S[16 x 32] = Q K^T over the
// whole row [c | k_rot] (zero-padded to a multiple of 64; the rows of the next chunk arrive by asynchronous copies
// meanwhile), warp w taking keys 8 (w % 4) .. and half of the k range;
// the two halves meet in shared memory where warp w takes the softmax step of rows w and w + 8 in 32-bit; the weights
// go back as two bfloat16 terms (p = hi + lo, so that the 32-bit weights lose nothing in the product); then
// O[16 x rank] += P C with warp w owning 8 NT latent columns, its accumulators in registers for the whole walk.
// NT: 8-column tiles a warp owns (rank = 64 NT).  Queries are rounded to bfloat16 (the product's left operand).
constexpr int LM_ROWS = 16;
constexpr int LM_PP = LA_KC + 8;           // row pitch of the weights (bfloat16)

template <int NT>
__global__ void __launch_bounds__(LA_THREADS)
latent_attention_mma_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot,
                            const float* __restrict__ sink, const __nv_bfloat16* __restrict__ cache,
                            const int32_t* __restrict__ block_table, int table_width,
                            const int32_t* __restrict__ token_req, const int32_t* __restrict__ positions,
                            __nv_bfloat16* lat, float* partial, int Tn, int H, int dr, int rank, int page_size,
                            int total_pages, int window, float scale, int n_splits, int* err) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    // (a long kernel, launched in the ordinary way: its blocks are placed when the machine is free, and the
    // kernel after it is let in only when it ends)
    typedef __nv_bfloat16 bf16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int width = rank + dr;
    const int wk = (width + 63) & ~63;                      // k extent of the score product
    const int qp = wk + 8;                                  // row pitch: 16 bytes off a multiple of 128
    bf16* s_q = reinterpret_cast<bf16*>(smem_raw);          // [16][qp]  queries [through W_uk | rotated part]
    bf16* s_keys0 = s_q + (size_t)LM_ROWS * qp;             // [2][32][qp]  the cache rows of this chunk and the next
    bf16* s_pb = s_keys0 + (size_t)2 * LA_KC * qp;          // [2][16][LM_PP] weights, high and low term
    float* s_s = reinterpret_cast<float*>(s_pb + 2 * LM_ROWS * LM_PP);   // [2][16][32] scores of the two k halves
    float* s_m = s_s + 2 * LM_ROWS * LA_KC;                 // [16]
    float* s_l = s_m + LM_ROWS;
    float* s_corr = s_l + LM_ROWS;
    const int t = blockIdx.x;
    const int h0 = blockIdx.y * LM_ROWS;
    const int hg = min(LM_ROWS, H - h0);
    const int ks_id = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int p = positions[t];
    for (int idx = threadIdx.x; idx < LM_ROWS * qp; idx += LA_THREADS) {
        const int row = idx / qp, c = idx - row * qp;
        float v = 0.f;
        if (row < hg) {
            if (c < rank) v = q_lat[((long long)(h0 + row) * Tn + t) * rank + c];
            else if (c < width) v = q_rot[((long long)t * H + h0 + row) * dr + (c - rank)];
        }
        s_q[idx] = __float2bfloat16_rn(v);
    }
    for (int idx = threadIdx.x; idx < 2 * LA_KC * (qp - width); idx += LA_THREADS) {     // the padding stays zero
        const int row = idx / (qp - width), c = idx - row * (qp - width);
        s_keys0[(size_t)row * qp + width + c] = __float2bfloat16_rn(0.f);
    }
    if (threadIdx.x < LM_ROWS) {
        s_m[threadIdx.x] = -INFINITY;
        s_l[threadIdx.x] = 0.f;
    }
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

    const int req = token_req[t];
    const int32_t* table = block_table + (long long)req * table_width;
    const int lo = window > 0 ? max(p - window + 1, 0) : 0;
    const int c_first = lo / LA_KC, c_last = p / LA_KC;
    const int per = (c_last - c_first + 1 + n_splits - 1) / n_splits;
    const int c_begin = c_first + ks_id * per, c_end = min(c_begin + per, c_last + 1);
    const int arow = (lane & 7) + 8 * ((lane >> 3) & 1);    // the row a lane names in a 16-row ldmatrix.x4
    const int n_base = warp * NT * 8;
    // the rows of chunk `ch` into buffer `which`: asynchronous 16-byte copies (zeros where the token sees no key)
    auto stage = [&](int ch, int which) {
        bf16* base = s_keys0 + (size_t)which * LA_KC * qp;
        for (int jj = warp; jj < LA_KC; jj += LA_THREADS / 32) {
            const int j = ch * LA_KC + jj;
            bf16* dst = base + (size_t)jj * qp;
            const bf16* row = nullptr;
            if (j >= lo && j <= p) {
                const int lp = j / page_size;
                const int page = lp < table_width ? table[lp] : -1;
                if (page < 0 || page >= total_pages) {
                    if (lane == 0) *err = 3;
                } else {
                    row = cache + ((long long)page * page_size + (j - lp * page_size)) * width;
                }
            }
            if (row == nullptr) {
                uint4* d4 = reinterpret_cast<uint4*>(dst);
                for (int i = lane; i < width / 8; i += 32) d4[i] = make_uint4(0u, 0u, 0u, 0u);
            } else {
                for (int i = lane; i < width / 8; i += 32) cp_async16(dst + 8 * i, row + 8 * i);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (c_begin < c_end) stage(c_begin, 0);
    for (int ch = c_begin; ch < c_end; ++ch) {
        const bf16* s_keys = s_keys0 + (size_t)((ch - c_begin) & 1) * LA_KC * qp;
        __syncthreads();                                    // the chunk before is done with the other buffer, s_s and s_pb
        if (ch + 1 < c_end) {
            stage(ch + 1, (ch + 1 - c_begin) & 1);          // the next chunk comes in while this one is worked on
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        // ---- scores: keys 8 nt .. 8 nt + 7, one half of the k range
        {
            const int nt = warp & 3, kh = warp >> 2;
            const int half = wk / 32;                       // k steps of 16 in a half (even: wk is a multiple of 64)
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const bf16* abase = s_q + (size_t)arow * qp + 8 * (lane >> 4);
            const bf16* bbase = s_keys + (size_t)(8 * nt + (lane & 7)) * qp + 8 * (lane >> 3);
            for (int ks = kh * half; ks < (kh + 1) * half; ks += 2) {
                uint32_t a0[4], a1[4], b[4];
                ldsm_x4(a0, abase + ks * 16);
                ldsm_x4(a1, abase + (ks + 1) * 16);
                ldsm_x4(b, bbase + ks * 16);                // k step ks (two halves), k step ks + 1 (two halves)
                mma16816(c, a0, b[0], b[1]);
                mma16816(c, a1, b[2], b[3]);
            }
            float* dst = s_s + kh * LM_ROWS * LA_KC;
            dst[g * LA_KC + 8 * nt + 2 * tq] = c[0];
            dst[g * LA_KC + 8 * nt + 2 * tq + 1] = c[1];
            dst[(g + 8) * LA_KC + 8 * nt + 2 * tq] = c[2];
            dst[(g + 8) * LA_KC + 8 * nt + 2 * tq + 1] = c[3];
        }
        __syncthreads();
        // ---- softmax step of rows warp and warp + 8 (lane = key)
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int row = warp + 8 * rr;
            const int j = ch * LA_KC + lane;
            float sc = (s_s[row * LA_KC + lane] + s_s[LM_ROWS * LA_KC + row * LA_KC + lane]) * scale;
            if (j < lo || j > p) sc = -INFINITY;
            const float m_old = s_m[row];
            const float m_new = fmaxf(m_old, warp_max(sc));
            float pw = 0.f, corr = 1.f;
            if (m_new > -INFINITY) {
                pw = expf(sc - m_new);
                corr = expf(m_old - m_new);
            }
            const float sum = warp_sum(pw);
            const bf16 hi = __float2bfloat16_rn(pw);
            s_pb[row * LM_PP + lane] = hi;
            s_pb[LM_ROWS * LM_PP + row * LM_PP + lane] = __float2bfloat16_rn(pw - __bfloat162float(hi));
            if (lane == 0) {
                s_l[row] = s_l[row] * corr + sum;
                s_m[row] = m_new;
                s_corr[row] = corr;
            }
        }
        __syncthreads();
        // ---- weighted latents: this warp's columns
        {
            const float c0 = s_corr[g], c1 = s_corr[g + 8];
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                acc[n][0] *= c0; acc[n][1] *= c0; acc[n][2] *= c1; acc[n][3] *= c1;
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                uint32_t ah[4], al[4];
                const bf16* pa = s_pb + arow * LM_PP + kk * 16 + 8 * (lane >> 4);
                ldsm_x4(ah, pa);
                ldsm_x4(al, pa + LM_ROWS * LM_PP);
                const bf16* kb = s_keys + (size_t)(kk * 16 + arow) * qp + n_base + 8 * (lane >> 4);
#pragma unroll
                for (int n = 0; n < NT; n += 2) {
                    uint32_t b[4];
                    ldsm_x4_trans(b, kb + n * 8);
                    mma16816(acc[n], ah, b[0], b[1]);
                    mma16816(acc[n], al, b[0], b[1]);
                    mma16816(acc[n + 1], ah, b[2], b[3]);
                    mma16816(acc[n + 1], al, b[2], b[3]);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int row = g + 8 * rr;
        if (row >= hg) continue;
        if (n_splits > 1) {
            float* dst = partial + (((long long)t * H + h0 + row) * n_splits + ks_id) * (rank + 2);
            if (warp == 0 && tq == 0) {
                dst[0] = s_m[row];
                dst[1] = s_l[row];
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                dst[2 + n_base + n * 8 + 2 * tq] = acc[n][2 * rr];
                dst[2 + n_base + n * 8 + 2 * tq + 1] = acc[n][2 * rr + 1];
            }
        } else {
            const float snk = sink ? sink[h0 + row] : -INFINITY;
            const float mm = fmaxf(s_m[row], snk);
            const float f = s_l[row] > 0.f ? expf(s_m[row] - mm) : 0.f;
            const float den = s_l[row] * f + (sink ? expf(snk - mm) : 0.f);
            const float w = den > 0.f ? f / den : 0.f;
            bf16* dst = lat + ((long long)(h0 + row) * Tn + t) * rank;
#pragma unroll
            for (int n = 0; n < NT; ++n)
                *reinterpret_cast<uint32_t*>(dst + n_base + n * 8 + 2 * tq) =
                    pack_bf16(acc[n][2 * rr] * w, acc[n][2 * rr + 1] * w);
        }
    }
}

// Merges the splits of a (token, head) in order and normalises as above.  One block a (token, head).
template <typename T>
__global__ void latent_merge_kernel(const float* __restrict__ partial, int n_splits, const float* __restrict__ sink,
                                    T* lat, int Tn, int H, int rank) {
    dep_wait();          // nothing is read or written before the kernels before this one have ended
    dep_launch_next();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* base = partial + ((long long)t * H + h) * n_splits * (rank + 2);
    const float snk = sink ? sink[h] : -INFINITY;
    float mm = snk;
    for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, base[(long long)s * (rank + 2)]);
    float den = sink ? expf(snk - mm) : 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float* ps = base + (long long)s * (rank + 2);
        if (ps[1] > 0.f) den += ps[1] * expf(ps[0] - mm);
    }
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    T* dst = lat + ((long long)h * Tn + t) * rank;
    for (int r = threadIdx.x; r < rank; r += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float* ps = base + (long long)s * (rank + 2);
            if (ps[1] > 0.f) v = fmaf(ps[2 + r], expf(ps[0] - mm), v);
        }
        dst[r] = from_f32<T>(v * inv);
    }
}

}  // namespace

void latent_prep(const float* proj, int ld, int off_q, int q_rank, const float* qn_w, int off_kv, int rank,
                 const float* kvn_w, int dr, const float* inv_freq, int rot_dims, int interleaved, const int32_t* positions,
                 const int32_t* slots, float eps, void* cq_out, void* cache, int page_size, int total_pages, int T,
                 int dtype, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= dr, "latent_prep: rotated dims must be even and <= dr");
    int* err = error_flag_ptr();
    if (dtype == F32)
        launch_dep(latent_prep_kernel<float>, dim3(T), dim3(128), 0, stream, proj, ld, off_q, q_rank, qn_w, off_kv, rank, kvn_w, dr, inv_freq,
                                                        rot_dims, interleaved, positions, slots, eps, static_cast<float*>(cq_out),
                                                        static_cast<float*>(cache), page_size, total_pages, err);
    else
        launch_dep(latent_prep_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, 
            proj, ld, off_q, q_rank, qn_w, off_kv, rank, kvn_w, dr, inv_freq, rot_dims, interleaved, positions, slots, eps,
            static_cast<__nv_bfloat16*>(cq_out), static_cast<__nv_bfloat16*>(cache), page_size, total_pages, err);
    check_launch("latent_prep");
}

namespace {
int heads_per_block(int H) {
    const int groups = (H + LA_HG - 1) / LA_HG;
    return (H + groups - 1) / groups;
}

template <typename T, int NCOL>
void launch_latent(const float* q_lat, const float* q_rot, const float* sink, const void* cache,
                   const int32_t* block_table, int table_width, const int32_t* token_req, const int32_t* positions,
                   void* lat, float* partial, int n_splits, int Tn, int H, int dr, int rank, int page_size,
                   int total_pages, int window, float scale, cudaStream_t stream) {
    const int hg = heads_per_block(H);
    const int wpad = (rank + dr + 7) & ~7;
    const size_t smem = ((size_t)LA_HG * (rank + dr) + LA_HG * LA_KC + 3 * LA_HG) * sizeof(float) +
                        (size_t)LA_KC * wpad * sizeof(T);
    DLM_CHECK(smem <= 220 * 1024, "latent_attention: sizes too large for shared memory");
    auto kern = latent_attention_kernel<T, NCOL>;
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        allowed = smem;
    }
    kern<<<dim3(Tn, (H + hg - 1) / hg, n_splits), LA_THREADS, smem, stream>>>(
        q_lat, q_rot, sink, static_cast<const T*>(cache), block_table, table_width, token_req, positions,
        static_cast<T*>(lat), partial, Tn, H, dr, rank, page_size, total_pages, window, scale, hg, n_splits,
        error_flag_ptr());
    check_launch("latent_attention");
    if (n_splits > 1) {
        launch_dep(latent_merge_kernel<T>, dim3(Tn, H), dim3(128), 0, stream, partial, n_splits, sink, static_cast<T*>(lat), Tn, H, rank);
        check_launch("latent_merge");
    }
}
}  // namespace

// The tensor-core kernel takes bfloat16 with a latent of 128, 256, 384 or 512 and a rotated part in multiples of 8
// (DLM_B200_NO_LATENT_MMA=1 switches it off).
bool latent_use_mma(int dtype, int rank, int dr, int fast) {
    static int off = -1;
    if (off < 0) {
        const char* e = std::getenv("DLM_B200_NO_LATENT_MMA");
        off = (e != nullptr && e[0] != '\0' && e[0] != '0') ? 1 : 0;
    }
    return fast && !off && dtype == BF16 && rank % 128 == 0 && rank <= 512 && dr % 8 == 0;
}

int latent_attention_splits(int T, int H, int rank, int dr, int max_keys, int dtype, int fast) {
    if (dtype == F32 || T <= 0) return 1;       // 32-bit: one order of summation whatever the step holds
    const int blocks = latent_use_mma(dtype, rank, dr, fast)
                           ? T * ((H + LM_ROWS - 1) / LM_ROWS)
                           : T * ((H + heads_per_block(H) - 1) / heads_per_block(H));
    int want = (2 * sm_count() + blocks - 1) / blocks;
    const int chunks = (max_keys < 1 ? 1 : max_keys) / LA_KC + 1;
    if (want > chunks) want = chunks;
    if (want > 32) want = 32;
    return want < 1 ? 1 : want;
}

void latent_q_split(const float* q, int ldq, const int32_t* positions, const float* inv_freq, int rot_dims,
                    int interleaved, void* qn, float* qr, int T, int H, int dn, int dr, int dtype, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(rot_dims % 2 == 0 && rot_dims >= 0 && rot_dims <= dr, "latent_q_split: rotated dims must be even and <= dr");
    if (dtype == F32)
        launch_dep(latent_q_split_kernel<float>, dim3(T), dim3(256), 0, stream, q, ldq, positions, inv_freq, rot_dims, interleaved, static_cast<float*>(qn),
                                                           qr, T, H, dn, dr);
    else
        launch_dep(latent_q_split_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, q, ldq, positions, inv_freq, rot_dims, interleaved,
                                                                   static_cast<__nv_bfloat16*>(qn), qr, T, H, dn, dr);
    check_launch("latent_q_split");
}

void latent_gate_out(const float* val, const float* gate, int ldg, void* out, int T, int H, int dv, int dtype,
                     cudaStream_t stream) {
    if (T <= 0) return;
    if (dtype == F32)
        launch_dep(latent_gate_out_kernel<float>, dim3(T), dim3(256), 0, stream, val, gate, ldg, static_cast<float*>(out), T, H, dv);
    else
        launch_dep(latent_gate_out_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, val, gate, ldg, static_cast<__nv_bfloat16*>(out), T,
                                                                    H, dv);
    check_launch("latent_gate_out");
}

void latent_attention(const float* q_lat, const float* q_rot, const float* sink, const void* cache,
                      const int32_t* block_table, int table_width, const int32_t* token_req, const int32_t* positions,
                      void* lat, float* partial, int n_splits, int T, int H, int dr, int rank, int page_size,
                      int total_pages, int window, float scale, int dtype, int fast, cudaStream_t stream) {
    if (T <= 0) return;
    DLM_CHECK(rank >= 1 && rank <= 1024, "latent_attention: latent size 1..1024");
    DLM_CHECK(n_splits >= 1 && (n_splits == 1 || partial != nullptr), "latent_attention: splits need a scratch buffer");
    if (latent_use_mma(dtype, rank, dr, fast)) {
        const int wk = (rank + dr + 63) & ~63, qp = wk + 8;
        const size_t smem = ((size_t)(LM_ROWS + 2 * LA_KC) * qp + 2 * LM_ROWS * LM_PP) * sizeof(__nv_bfloat16) +
                            (2 * LM_ROWS * LA_KC + 3 * LM_ROWS) * sizeof(float);
        const dim3 grid(T, (H + LM_ROWS - 1) / LM_ROWS, n_splits);
#define DLM_LMMA(NT)                                                                                                  \
    do {                                                                                                              \
        auto kern = latent_attention_mma_kernel<NT>;                                                                  \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
        kern<<<grid, LA_THREADS, smem, stream>>>(q_lat, q_rot, sink, static_cast<const __nv_bfloat16*>(cache),        \
                                                 block_table, table_width, token_req, positions,                      \
                                                 static_cast<__nv_bfloat16*>(lat), partial, T, H, dr, rank, page_size, \
                                                 total_pages, window, scale, n_splits, error_flag_ptr());             \
    } while (0)
        switch (rank / 64) {
            case 2: DLM_LMMA(2); break;
            case 4: DLM_LMMA(4); break;
            case 6: DLM_LMMA(6); break;
            default: DLM_LMMA(8); break;
        }
#undef DLM_LMMA
        check_launch("latent_attention (tensor cores)");
        if (n_splits > 1) {
            launch_dep(latent_merge_kernel<__nv_bfloat16>, dim3(T, H), dim3(128), 0, stream, 
                partial, n_splits, sink, static_cast<__nv_bfloat16*>(lat), T, H, rank);
            check_launch("latent_merge");
        }
        return;
    }
#define DLM_LAT(TT, NC)                                                                                               \
    launch_latent<TT, NC>(q_lat, q_rot, sink, cache, block_table, table_width, token_req, positions, lat, partial,    \
                          n_splits, T, H, dr, rank, page_size, total_pages, window, scale, stream)
    const int nc = (rank + LA_THREADS - 1) / LA_THREADS;
    if (dtype == F32) {
        if (nc <= 1) DLM_LAT(float, 1);
        else if (nc <= 2) DLM_LAT(float, 2);
        else DLM_LAT(float, 4);
    } else {
        if (nc <= 1) DLM_LAT(__nv_bfloat16, 1);
        else if (nc <= 2) DLM_LAT(__nv_bfloat16, 2);
        else DLM_LAT(__nv_bfloat16, 4);
    }
#undef DLM_LAT
}

}  // namespace dlmk
