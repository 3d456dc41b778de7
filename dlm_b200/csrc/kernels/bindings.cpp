// Python bindings of the kernel launchers.  Pointers and the stream arrive as integers
// (tensor.data_ptr(), stream.cuda_stream); shapes are checked on the Python side.
#include <pybind11/pybind11.h>

#include "api.h"

namespace py = pybind11;
using u64 = uintptr_t;

namespace {
template <typename T> T* ptr(u64 p) { return reinterpret_cast<T*>(p); }
cudaStream_t st(u64 s) { return reinterpret_cast<cudaStream_t>(s); }
}  // namespace

PYBIND11_MODULE(_dlm_kernels, m) {
    m.doc() = "dlm_b200 sm_100a kernels";
    m.attr("EPI_STORE") = (int)dlmk::EPI_STORE;
    m.attr("EPI_ADD") = (int)dlmk::EPI_ADD;
    m.attr("EPI_SWIGLU") = (int)dlmk::EPI_SWIGLU;
    m.attr("EPI_GELU") = (int)dlmk::EPI_GELU;
    m.attr("EPI_GELU_TANH") = (int)dlmk::EPI_GELU_TANH;

    m.def("embed", [](u64 tokens, u64 table, u64 out, int T, int H, int V, float scale, int dtype, u64 stream) {
        dlmk::embed(ptr<const int32_t>(tokens), ptr<const void>(table), ptr<float>(out), T, H, V, scale, dtype,
                    st(stream));
    });
    m.def("rmsnorm", [](u64 x, u64 w, u64 out, u64 rows, int n_rows, int H, float eps, int out_dtype, u64 stream) {
        dlmk::rmsnorm(ptr<const float>(x), ptr<const float>(w), ptr<void>(out), ptr<const int32_t>(rows), n_rows, H,
                      eps, out_dtype, st(stream));
    });
    m.def("gemm", [](u64 a, int lda, u64 a_rows, u64 w, int ldw, long long w_expert_stride, u64 expert_offsets,
                     int num_experts, u64 bias, u64 out, int ldo, int M, int N, int K, int in_dtype, int out_dtype,
                     int epilogue, int fast, u64 stream) {
        dlmk::gemm(ptr<const void>(a), lda, ptr<const int32_t>(a_rows), ptr<const void>(w), ldw, w_expert_stride,
                   ptr<const int32_t>(expert_offsets), num_experts, ptr<const float>(bias), ptr<void>(out), ldo, M, N,
                   K, in_dtype, out_dtype, epilogue, fast, st(stream));
    });
    m.def("rope_kv_write", [](u64 qkv, u64 positions, u64 inv_freq, int rotary_dim, int interleaved, u64 slots,
                              u64 q_out, u64 k_cache, u64 v_cache, int T, int nh, int nkv, int hd, int page_size,
                              int total_pages, int dtype, u64 stream) {
        dlmk::rope_kv_write(ptr<const float>(qkv), ptr<const int32_t>(positions), ptr<const float>(inv_freq),
                            rotary_dim, interleaved, ptr<const int32_t>(slots), ptr<void>(q_out), ptr<void>(k_cache),
                            ptr<void>(v_cache), T, nh, nkv, hd, page_size, total_pages, dtype, st(stream));
    });
    m.def("attention", [](u64 q, u64 k_cache, u64 v_cache, u64 block_table, int table_width, u64 cu_q, u64 kv_len,
                          u64 out, int T, int R, int nh, int nkv, int hd, int page_size, int total_pages, int window,
                          float scale, u64 slopes, int chunk, u64 sinks, float softcap, int max_q_len, int max_kv_len,
                          int num_single, u64 scratch, int dtype, int fast, u64 stream) {
        dlmk::attention(ptr<const void>(q), ptr<const void>(k_cache), ptr<const void>(v_cache),
                        ptr<const int32_t>(block_table), table_width, ptr<const int32_t>(cu_q),
                        ptr<const int32_t>(kv_len), ptr<void>(out), T, R, nh, nkv, hd, page_size, total_pages, window,
                        scale, ptr<const float>(slopes), chunk, ptr<const float>(sinks), softcap, max_q_len, max_kv_len,
                        num_single, ptr<float>(scratch), dtype, fast, st(stream));
    });
    m.def("attention_scratch_floats", [](int R, int nh, int nkv, int hd, int max_kv_len) {
        return dlmk::attention_scratch_floats(R, nh, nkv, hd, max_kv_len);
    });
    m.def("router_topk", [](u64 h, u64 w, u64 norm_w, float eps, u64 logits, u64 ids, u64 wts, u64 gate, int T, int H,
                            int E, int k, int norm, int has_gate, int dtype, int h_is_f32, int score_fn, float scale,
                            u64 select_bias, u64 stream) {
        dlmk::router_topk(ptr<const void>(h), ptr<const void>(w), ptr<const float>(norm_w), eps, ptr<float>(logits),
                          ptr<int32_t>(ids), ptr<float>(wts), ptr<float>(gate), T, H, E, k, norm, has_gate, dtype,
                          h_is_f32, score_fn, scale, ptr<const float>(select_bias), 0, st(stream));
    });
    m.def("router_topk_permute", [](u64 h, u64 w, u64 norm_w, float eps, u64 logits, u64 ids, u64 wts, u64 gate,
                                    u64 offsets, u64 rows, u64 dest, int T, int H, int E, int k, int norm, int has_gate,
                                    int dtype, int h_is_f32, int score_fn, float scale, u64 select_bias, int x_settled,
                                    u64 stream) {
        return dlmk::router_topk_permute(ptr<const void>(h), ptr<const void>(w), ptr<const float>(norm_w), eps,
                                  ptr<float>(logits), ptr<int32_t>(ids), ptr<float>(wts), ptr<float>(gate),
                                  ptr<int32_t>(offsets), ptr<int32_t>(rows), ptr<int32_t>(dest), T, H, E, k, norm,
                                  has_gate, dtype, h_is_f32, score_fn, scale, ptr<const float>(select_bias),
                                  x_settled, st(stream));
    });
    m.def("moe_permute", [](u64 ids, int n, int k, int E, u64 offsets, u64 rows, u64 dest, u64 stream) {
        dlmk::moe_permute(ptr<const int32_t>(ids), n, k, E, ptr<int32_t>(offsets), ptr<int32_t>(rows),
                          ptr<int32_t>(dest), st(stream));
    });
    m.def("moe_combine", [](u64 y, u64 dest, u64 wts, u64 shared, u64 gate, u64 resid, int T, int H, int k, u64 ids,
                            int num_real, u64 passthrough, float shared_scale, u64 stream) {
        dlmk::moe_combine(ptr<const float>(y), ptr<const int32_t>(dest), ptr<const float>(wts),
                          ptr<const float>(shared), ptr<const float>(gate), ptr<float>(resid), T, H, k,
                          ptr<const int32_t>(ids), num_real, ptr<const float>(passthrough), shared_scale, st(stream));
    });
    m.def("argmax", [](u64 logits, u64 out, int N, int V, u64 scratch, u64 stream) {
        dlmk::argmax(ptr<const float>(logits), ptr<int32_t>(out), N, V, ptr<void>(scratch), st(stream));
    });
    m.def("argmax_scratch_bytes", [](int N, int V) { return dlmk::argmax_scratch_bytes(N, V); });
    m.def("sample", [](u64 logits, u64 out, int N, int V, u64 params, u64 top_k, u64 u, u64 seen_offsets,
                       u64 seen_tokens, u64 scratch, u64 stream) {
        dlmk::sample(ptr<const float>(logits), ptr<int32_t>(out), N, V, ptr<const float>(params),
                     ptr<const int32_t>(top_k), ptr<const float>(u), ptr<const int32_t>(seen_offsets),
                     ptr<const int32_t>(seen_tokens), ptr<float>(scratch), st(stream));
    });
    m.def("gemm_tc_enabled", &dlmk::gemm_tc_enabled);
    m.def("gather_rows", [](u64 src, u64 rows, u64 out, int n_rows, int width, int dtype, u64 stream) {
        dlmk::gather_rows(ptr<const void>(src), ptr<const int32_t>(rows), ptr<void>(out), n_rows, width, dtype,
                          st(stream));
    });
    m.def("add_rows", [](u64 x, u64 table, u64 idx, int T, int H, int rows, int dtype, u64 stream) {
        dlmk::add_rows(ptr<float>(x), ptr<const void>(table), ptr<const int32_t>(idx), T, H, rows, dtype, st(stream));
    });
    m.def("streams_expand", [](u64 x, u64 xs, int T, int S, int H, u64 stream) {
        dlmk::streams_expand(ptr<const float>(x), ptr<float>(xs), T, S, H, st(stream));
    });
    m.def("streams_reduce", [](u64 xs, u64 a, u64 norm_w, float eps, u64 out, int T, int S, int H, int out_dtype,
                               u64 stream) {
        dlmk::streams_reduce(ptr<const float>(xs), ptr<const float>(a), ptr<const float>(norm_w), eps, ptr<void>(out), T,
                             S, H, out_dtype, st(stream));
    });
    m.def("streams_update", [](u64 xs, u64 mix, u64 outw, u64 y, int T, int S, int H, u64 stream) {
        dlmk::streams_update(ptr<float>(xs), ptr<const float>(mix), ptr<const float>(outw), ptr<const float>(y), T, S, H,
                             st(stream));
    });
    m.def("streams_update_reduce", [](u64 xs, u64 mix, u64 outw, u64 y, u64 in_next, u64 norm_w, float eps, u64 out, int T,
                                      int S, int H, int out_dtype, u64 stream) {
        dlmk::streams_update_reduce(ptr<float>(xs), ptr<const float>(mix), ptr<const float>(outw), ptr<const float>(y),
                                    ptr<const float>(in_next), ptr<const float>(norm_w), eps, ptr<void>(out), T, S, H,
                                    out_dtype, st(stream));
    });
    m.def("causal_conv", [](u64 x, int ldx, u64 w, u64 bias, u64 state, u64 cu_q, u64 token_req, u64 state_slot, int T,
                            int R, int C, int taps, int add_input, int act, u64 out, int ldo, int out_dtype, u64 stream) {
        dlmk::causal_conv(ptr<const float>(x), ldx, ptr<const float>(w), ptr<const float>(bias), ptr<float>(state),
                          ptr<const int32_t>(cu_q), ptr<const int32_t>(token_req), ptr<const int32_t>(state_slot), T, R,
                          C, taps, add_input, act, ptr<void>(out), ldo, out_dtype, st(stream));
    });
    m.def("activation", [](u64 x, int ldx, u64 out, int ldo, int rows, int cols, int op, int out_dtype, u64 stream) {
        dlmk::activation(ptr<const float>(x), ldx, ptr<void>(out), ldo, rows, cols, op, out_dtype, st(stream));
    });
    m.def("table_lookup", [](u64 tokens, u64 table, u64 ids, u64 wts, int T, int V, int top, int E, u64 stream) {
        dlmk::table_lookup(ptr<const int32_t>(tokens), ptr<const int32_t>(table), ptr<int32_t>(ids), ptr<float>(wts), T,
                           V, top, E, st(stream));
    });
    m.def("gated_rmsnorm", [](u64 y, int ldy, u64 gate, int ldg, u64 w, u64 out, int ldo, int T, int groups,
                              int group_size, float eps, int mode, int out_dtype, u64 row_scale, u64 stream) {
        dlmk::gated_rmsnorm(ptr<const float>(y), ldy, ptr<const float>(gate), ldg, ptr<const float>(w), ptr<void>(out),
                            ldo, T, groups, group_size, eps, mode, out_dtype, ptr<const float>(row_scale), st(stream));
    });
    m.def("ssm_scan", [](u64 xbc, int ldx, u64 dt_raw, int lddt, u64 dt_bias, u64 A_log, u64 D, u64 state, u64 cu_q,
                         u64 state_slot, u64 y, int R, int heads, int P, int N, int groups, u64 fixed_decay,
                         u64 stream) {
        dlmk::ssm_scan(ptr<const float>(xbc), ldx, ptr<const float>(dt_raw), lddt, ptr<const float>(dt_bias),
                       ptr<const float>(A_log), ptr<const float>(D), ptr<float>(state), ptr<const int32_t>(cu_q),
                       ptr<const int32_t>(state_slot), ptr<float>(y), R, heads, P, N, groups,
                       ptr<const float>(fixed_decay), st(stream));
    });
    m.def("delta_scan", [](u64 proj, int ld, int off_r, int off_k, int off_v, int off_a, u64 lw, int ldlw, u64 a_bias,
                           u64 state, u64 cu_q, u64 state_slot, u64 o, int R, int heads, int d, float unit_eps,
                           float decay_coef, u64 stream) {
        dlmk::delta_scan(ptr<const float>(proj), ld, off_r, off_k, off_v, off_a, ptr<const float>(lw), ldlw,
                         ptr<const float>(a_bias), ptr<float>(state), ptr<const int32_t>(cu_q),
                         ptr<const int32_t>(state_slot), ptr<float>(o), R, heads, d, unit_eps, decay_coef, st(stream));
    });
    m.def("selective_scan", [](u64 x, int ldx, u64 dt_raw, int lddt, u64 bc, int ldbc, u64 z, int ldz, u64 dt_bias, u64 A_log,
                               u64 D, u64 state, u64 cu_q, u64 state_slot, u64 out, int ldo, int R, int inner, int N,
                               int out_dtype, u64 stream) {
        dlmk::selective_scan(ptr<const float>(x), ldx, ptr<const float>(dt_raw), lddt, ptr<const float>(bc), ldbc,
                             ptr<const float>(z), ldz, ptr<const float>(dt_bias), ptr<const float>(A_log),
                             ptr<const float>(D), ptr<float>(state), ptr<const int32_t>(cu_q),
                             ptr<const int32_t>(state_slot), ptr<void>(out), ldo, R, inner, N, out_dtype, st(stream));
    });
    m.def("qk_norm_write", [](u64 qkv, int ld, u64 positions, u64 qn_w, u64 kn_w, float eps, float temp_coef,
                              int temp_every, u64 slots, u64 q_out, u64 k_cache, u64 v_cache, int T, int nh, int nkv,
                              int d, int dv, int D, int page_size, int total_pages, int dtype, u64 stream) {
        dlmk::qk_norm_write(ptr<const float>(qkv), ld, ptr<const int32_t>(positions), ptr<const float>(qn_w),
                            ptr<const float>(kn_w), eps, temp_coef, temp_every, ptr<const int32_t>(slots),
                            ptr<void>(q_out), ptr<void>(k_cache), ptr<void>(v_cache), T, nh, nkv, d, dv, D, page_size,
                            total_pages, dtype, st(stream));
    });
    m.def("rotate_heads", [](u64 x, int ld, u64 positions, u64 inv_freq, int rot_dims, int T, int heads, int dim,
                             int off_a, float scale_a, int off_b, float scale_b, u64 stream) {
        dlmk::rotate_heads(ptr<float>(x), ld, ptr<const int32_t>(positions), ptr<const float>(inv_freq), rot_dims, T,
                           heads, dim, off_a, scale_a, off_b, scale_b, st(stream));
    });
    m.def("branch_norm_add", [](u64 resid, u64 a, u64 wa, u64 b, u64 wb, float eps, float coef, int T, int H,
                                u64 stream) {
        dlmk::branch_norm_add(ptr<float>(resid), ptr<const float>(a), ptr<const float>(wa), ptr<const float>(b),
                              ptr<const float>(wb), eps, coef, T, H, st(stream));
    });
    m.def("rmsnorm_pair", [](u64 x, u64 wa, u64 wb, u64 out_a, u64 out_b, int T, int H, float eps, int out_dtype, u64 stream) {
        dlmk::rmsnorm_pair(ptr<const float>(x), ptr<const float>(wa), ptr<const float>(wb), ptr<void>(out_a),
                           ptr<void>(out_b), T, H, eps, out_dtype, st(stream));
    });
    m.def("concat_rows", [](u64 a, u64 b, u64 out, int T, int H, int out_dtype, u64 stream) {
        dlmk::concat_rows(ptr<const float>(a), ptr<const float>(b), ptr<void>(out), T, H, out_dtype, st(stream));
    });
    m.def("latent_prep", [](u64 proj, int ld, int off_q, int q_rank, u64 qn_w, int off_kv, int rank, u64 kvn_w, int dr,
                            u64 inv_freq, int rot_dims, int interleaved, u64 positions, u64 slots, float eps, u64 cq_out,
                            u64 cache, int page_size, int total_pages, int T, int dtype, u64 stream) {
        dlmk::latent_prep(ptr<const float>(proj), ld, off_q, q_rank, ptr<const float>(qn_w), off_kv, rank,
                          ptr<const float>(kvn_w), dr, ptr<const float>(inv_freq), rot_dims, interleaved,
                          ptr<const int32_t>(positions), ptr<const int32_t>(slots), eps, ptr<void>(cq_out),
                          ptr<void>(cache), page_size, total_pages, T, dtype, st(stream));
    });
    m.def("latent_q_split", [](u64 q, int ldq, u64 positions, u64 inv_freq, int rot_dims, int interleaved, u64 qn,
                               u64 qr, int T, int H, int dn, int dr, int dtype, u64 stream) {
        dlmk::latent_q_split(ptr<const float>(q), ldq, ptr<const int32_t>(positions), ptr<const float>(inv_freq), rot_dims,
                             interleaved, ptr<void>(qn), ptr<float>(qr), T, H, dn, dr, dtype, st(stream));
    });
    m.def("latent_gate_out", [](u64 val, u64 gate, int ldg, u64 out, int T, int H, int dv, int dtype, u64 stream) {
        dlmk::latent_gate_out(ptr<const float>(val), ptr<const float>(gate), ldg, ptr<void>(out), T, H, dv, dtype,
                              st(stream));
    });
    m.def("latent_attention", [](u64 q_lat, u64 q_rot, u64 sink, u64 cache, u64 block_table, int table_width,
                                 u64 token_req, u64 positions, u64 lat, u64 partial, int n_splits, int T, int H, int dr,
                                 int rank, int page_size, int total_pages, int window, float scale, int dtype, int fast,
                                 u64 stream) {
        dlmk::latent_attention(ptr<const float>(q_lat), ptr<const float>(q_rot), ptr<const float>(sink),
                               ptr<const void>(cache), ptr<const int32_t>(block_table), table_width,
                               ptr<const int32_t>(token_req), ptr<const int32_t>(positions), ptr<void>(lat),
                               ptr<float>(partial), n_splits, T, H, dr, rank, page_size, total_pages, window, scale, dtype,
                               fast, st(stream));
    });
    m.def("latent_attention_splits", &dlmk::latent_attention_splits);
    m.def("gated_scan", [](u64 q, int ldq, u64 k, int ldk, u64 v, int ldv, u64 dec, int ldd, u64 beta, int ldb, u64 A_log,
                           u64 dec_bias, u64 state, u64 cu_q, u64 state_slot, u64 o, int ldo, int R, int heads,
                           int qk_heads, int dk, int dv, int unit, float unit_eps, float q_scale, int decay_kind,
                           float tau, u64 stream) {
        dlmk::gated_scan(ptr<const float>(q), ldq, ptr<const float>(k), ldk, ptr<const float>(v), ldv,
                         ptr<const float>(dec), ldd, ptr<const float>(beta), ldb, ptr<const float>(A_log),
                         ptr<const float>(dec_bias), ptr<float>(state), ptr<const int32_t>(cu_q),
                         ptr<const int32_t>(state_slot), ptr<float>(o), ldo, R, heads, qk_heads, dk, dv, unit, unit_eps,
                         q_scale, decay_kind, tau, st(stream));
    });
    m.def("head_norm_rope_write", [](u64 qkv, int ld, u64 positions, u64 qn_w, u64 kn_w, float eps, u64 inv_freq,
                                     int rot_dims, int interleaved, u64 slots, u64 q_out, u64 k_cache, u64 v_cache, int T,
                                     int nh, int nkv, int d, int dv, int D, int page_size, int total_pages, int dtype,
                                     u64 stream) {
        dlmk::head_norm_rope_write(ptr<const float>(qkv), ld, ptr<const int32_t>(positions), ptr<const float>(qn_w),
                                   ptr<const float>(kn_w), eps, ptr<const float>(inv_freq), rot_dims, interleaved,
                                   ptr<const int32_t>(slots), ptr<void>(q_out), ptr<void>(k_cache), ptr<void>(v_cache), T,
                                   nh, nkv, d, dv, D, page_size, total_pages, dtype, st(stream));
    });
    m.def("head_gate", [](u64 o, u64 gate, int ldg, int T, int nh, int D, float factor, int dtype, u64 stream) {
        dlmk::head_gate(ptr<void>(o), ptr<const float>(gate), ldg, T, nh, D, factor, dtype, st(stream));
    });
    m.def("norm_add_norm", [](u64 resid, u64 y, u64 w_post, u64 w_next, float eps, u64 out, int T, int H, int out_dtype,
                              u64 stream) {
        dlmk::norm_add_norm(ptr<float>(resid), ptr<const float>(y), ptr<const float>(w_post), ptr<const float>(w_next),
                            eps, ptr<void>(out), T, H, out_dtype, st(stream));
    });
    m.def("add_vec_rows", [](u64 x, u64 x0, u64 vec, int T, int H, u64 stream) {
        dlmk::add_vec_rows(ptr<float>(x), ptr<const float>(x0), ptr<const float>(vec), T, H, st(stream));
    });
    m.def("memory_scan", [](u64 q, int ldq, u64 k, int ldk, u64 v, int ldv, u64 igate, int ldi, u64 fgate, int ldf,
                            u64 i_bias, u64 f_bias, float cap, u64 state, u64 nstate, u64 mstate, u64 cu_q, u64 state_slot,
                            u64 o, int ldo, u64 rden, int R, int heads, int dk, int dv, float q_scale, float den_eps,
                            u64 stream) {
        dlmk::memory_scan(ptr<const float>(q), ldq, ptr<const float>(k), ldk, ptr<const float>(v), ldv,
                          ptr<const float>(igate), ldi, ptr<const float>(fgate), ldf, ptr<const float>(i_bias),
                          ptr<const float>(f_bias), cap, ptr<float>(state), ptr<float>(nstate), ptr<float>(mstate),
                          ptr<const int32_t>(cu_q), ptr<const int32_t>(state_slot), ptr<float>(o), ldo, ptr<float>(rden),
                          R, heads, dk, dv, q_scale, den_eps, st(stream));
    });
    m.def("dyt_norm", [](u64 x, u64 rows, u64 w, u64 b, float alpha, u64 out, int n_rows, int H, int out_dtype,
                         u64 stream) {
        dlmk::dyt_norm(ptr<const float>(x), ptr<const int32_t>(rows), ptr<const float>(w), ptr<const float>(b), alpha,
                       ptr<void>(out), n_rows, H, out_dtype, st(stream));
    });
    m.def("dyt_norm_pair", [](u64 x, u64 wa, u64 ba, float alpha_a, u64 out_a, u64 wb, u64 bb, float alpha_b, u64 out_b,
                              u64 out_b32, int T, int H, int out_dtype, u64 stream) {
        dlmk::dyt_norm_pair(ptr<const float>(x), ptr<const float>(wa), ptr<const float>(ba), alpha_a, ptr<void>(out_a),
                            ptr<const float>(wb), ptr<const float>(bb), alpha_b, ptr<void>(out_b), ptr<float>(out_b32),
                            T, H, out_dtype, st(stream));
    });
    m.def("tanh_cap", [](u64 x, long long n, float cap, u64 stream) { dlmk::tanh_cap(ptr<float>(x), n, cap, st(stream)); });
    m.def("entry_gate", [](u64 o, u64 gate, int ldg, int T, int nh, int dv, int D, float factor, int dtype, u64 resid,
                           u64 bias, int W, u64 stream) {
        dlmk::entry_gate(ptr<void>(o), ptr<const float>(gate), ldg, T, nh, dv, D, factor, dtype, ptr<float>(resid),
                         ptr<const float>(bias), W, st(stream));
    });
    m.def("take_error_flag", &dlmk::take_error_flag);
    m.def("reset_decode_merge_counters", [](u64 stream) { dlmk::reset_decode_merge_counters(st(stream)); });
    m.def("dep_launch_enabled", &dlmk::dep_launch_enabled);
    m.def("set_dep_launch", &dlmk::set_dep_launch);
}
