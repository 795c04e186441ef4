/*
 * ref_cpu_shim.cpp -- C entry points around the UPSTREAM CPU kernels.  TEST INFRASTRUCTURE ONLY.
 *
 * oracle/build.py compiles this file together with the upstream source csrc/cpu/quant_cpu.cpp (taken from
 * an upstream checkout where it lies, not copied into this repository) against the installed torch
 * headers into oracle/_ref/libtq_ref_cpu.so.  The upstream functions take torch tensors; the shim wraps
 * raw host pointers into tensors (no copies) and drives them the way the upstream cache does for one
 * decode step: per (sequence, KV head) the logits of the group's query heads over the packed keys
 * (attention_scores_packed_cpu, quant_cpu.cpp:125-193), softmax, the weighted sum over the packed values
 * (attention_values_packed_cpu, quant_cpu.cpp:199-266).  The upstream kernels parallelise over the
 * (batch, head) pairs of ONE call -- four query heads here -- so the shim spreads the units over the
 * host threads with an OpenMP loop of its own; inside a unit the upstream code runs unchanged.
 */
#include <torch/torch.h>

#include <cstdint>
#include <cstring>

#ifdef _OPENMP
#include <omp.h>
#endif

/* upstream csrc/cpu/quant_cpu.cpp */
std::tuple<torch::Tensor, torch::Tensor> rotate_and_quantize_cpu(torch::Tensor vectors, torch::Tensor rotation,
                                                                 torch::Tensor boundaries, int64_t bit_width);
torch::Tensor attention_scores_packed_cpu(torch::Tensor query, torch::Tensor packed_keys, torch::Tensor key_norms,
                                          torch::Tensor centroids, torch::Tensor rotation, int64_t bit_width);
torch::Tensor attention_values_packed_cpu(torch::Tensor attn_weights, torch::Tensor packed_values,
                                          torch::Tensor value_norms, torch::Tensor centroids, torch::Tensor rotation_T,
                                          int64_t bit_width);

namespace {
torch::Tensor f32(const float* p, at::IntArrayRef shape) {
    return torch::from_blob(const_cast<float*>(p), shape, torch::kFloat32);
}
torch::Tensor u8(const uint8_t* p, at::IntArrayRef shape) {
    return torch::from_blob(const_cast<uint8_t*>(p), shape, torch::kUInt8);
}
}  // namespace

extern "C" {

__attribute__((visibility("default"))) int tqc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

__attribute__((visibility("default"))) void tqc_set_num_threads(int n) {
    // torch's own intra-op pool first (it sets the OpenMP thread count as a side effect), then the count for
    // the loop over units below: inside that loop torch's operators run on the unit's thread (nested regions
    // are serial).
    at::set_num_threads(n > 0 ? n : 1);
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#endif
}

/* rotate_and_quantize_cpu, quant_cpu.cpp:44-119: (n, dim) float32 -> packed codes and norms. */
__attribute__((visibility("default"))) int tqc_rotate_and_quantize(const float* x, int n, int dim, const float* rotation,
                                                                   const float* boundaries, int bits, uint8_t* packed,
                                                                   float* norms) {
    try {
        auto res = rotate_and_quantize_cpu(f32(x, {n, dim}), f32(rotation, {dim, dim}), f32(boundaries, {(1 << bits) - 1}), bits);
        auto p = std::get<0>(res).contiguous();
        auto nr = std::get<1>(res).contiguous();
        std::memcpy(packed, p.data_ptr<uint8_t>(), (size_t)p.numel());
        std::memcpy(norms, nr.data_ptr<float>(), (size_t)nr.numel() * sizeof(float));
        return 0;
    } catch (...) {
        return -1;
    }
}

/* One decode step over a packed cache in upstream row layout:
 *   query (batch, q_heads, dim); k_packed (batch, kv_heads, max_seq, pk), k_norms (batch, kv_heads, max_seq);
 *   values alike; lens (batch); out (batch, q_heads, dim).  inv_rot_v is the matrix M of
 *   attention_values_packed_cpu's last step, out = rotated @ M. */
__attribute__((visibility("default"))) int tqc_decode_attention(
    const float* query, const uint8_t* k_packed, const float* k_norms, const uint8_t* v_packed, const float* v_norms,
    const int32_t* lens, int batch, int q_heads, int kv_heads, int max_seq, int dim, int kbits, int vbits,
    const float* rot_k, const float* cent_k, const float* inv_rot_v, const float* cent_v, float scale, float* out) {
    const int group = q_heads / kv_heads;
    const int64_t pk = (int64_t)kbits * ((dim + 7) / 8), pv = (int64_t)vbits * ((dim + 7) / 8);
    int failed = 0;
#pragma omp parallel for schedule(dynamic) reduction(| : failed)
    for (int u = 0; u < batch * kv_heads; u++) {
        try {
            torch::NoGradGuard no_grad;
            const int b = u / kv_heads, h = u % kv_heads, len = lens[b];
            float* o = out + ((int64_t)b * q_heads + (int64_t)h * group) * dim;
            if (len <= 0) {
                std::memset(o, 0, sizeof(float) * group * dim);
                continue;
            }
            auto q = f32(query + ((int64_t)b * q_heads + (int64_t)h * group) * dim, {1, group, dim});
            auto logits = attention_scores_packed_cpu(q, u8(k_packed + (int64_t)u * max_seq * pk, {len, pk}),
                                                      f32(k_norms + (int64_t)u * max_seq, {len}),
                                                      f32(cent_k, {1 << kbits}), f32(rot_k, {dim, dim}), kbits);
            auto weights = torch::softmax(logits * scale, -1);
            auto res = attention_values_packed_cpu(weights, u8(v_packed + (int64_t)u * max_seq * pv, {len, pv}),
                                                   f32(v_norms + (int64_t)u * max_seq, {len}),
                                                   f32(cent_v, {1 << vbits}), f32(inv_rot_v, {dim, dim}), vbits)
                           .contiguous();
            std::memcpy(o, res.data_ptr<float>(), sizeof(float) * group * dim);
        } catch (...) {
            failed |= 1;
        }
    }
    return failed ? -1 : 0;
}

}  // extern "C"
