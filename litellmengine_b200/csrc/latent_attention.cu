// The small kernels of latent attention: attention whose keys and values are linear maps of one cached latent
// row per token.  Per token the pages hold ONE row [c | kr]: the normed latent c (R entries) and a rotated key
// part kr (P entries) that all heads share.  With the per-head maps folded into the query and the output
// (q_abs[h] = W_uk[h]^T q_nope[h], o[h] = W_uv[h] sum_j p_j c_j) attention runs straight over those rows: every
// head scores [q_abs[h] | q_rot[h]] against [c | kr], and sums the first R entries of the rows it attends to.
//
//   latent_prepare   from the float32 projection of the layer input, columns [dq | dkv]:
//                      cq = rmsnorm(dq) * wq                      -> [T, Q] in the compute dtype (feeds W_uq)
//                      c  = rmsnorm(dkv[:R]) * wkv,  kr = rotate(dkv[R:R+P])   -> the token's row in its page
//                    (the second half only for a layer that keeps its own latent).
//   latent_q_split   from q = W_uq cq (float32 [T, H*(D+P)], per head [D unrotated | P rotated]):
//                      qn[h, t, :] = q_nope in the compute dtype, head-major (the left operand of the batched
//                      product with W_uk), and the rotated q_rot into columns R .. R+P of head h of the packed
//                      query [T, H*(R+P)], whose first R columns per head that product then fills.
//
// Rotation: the first `dims` entries of the P-part, entry i paired with i + dims/2, by the angle
// float(position) * inv_freq[i], sine and cosine in 32-bit; the rest passes unchanged.  Norms are 32-bit.
#include "common.cuh"

#define LA_THREADS 256

template <typename TQ, typename TC>
__global__ void latent_prepare_kernel(
    const float* __restrict__ proj, long long proj_stride, int dq_off, int dkv_off, int Q, int R, int P, int dims,
    const float* __restrict__ wq, const float* __restrict__ wkv, float eps, const float* __restrict__ inv_freq,
    TQ* __restrict__ cq_out, TC* __restrict__ keys, long long key_page_stride,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table, int table_stride,
    int page_size, int num_pages, int32_t* __restrict__ status) {
    pdl_begin();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float* row = proj + static_cast<size_t>(t) * proj_stride;
    {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < Q; i += blockDim.x) { const float a = row[dq_off + i]; ss += a * a; }
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(Q) + eps);
        for (int i = threadIdx.x; i < Q; i += blockDim.x)
            cq_out[static_cast<size_t>(t) * Q + i] = from_f32<TQ>(row[dq_off + i] * inv * wq[i]);
    }
    if (!keys) return;
    const int pos = positions[t];
    const int slot = entry_slot[token_entry[t]];
    const int logical = pos / page_size;
    const int page = logical < table_stride ? block_table[static_cast<size_t>(slot) * table_stride + logical] : -1;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && atomicCAS(status, 0, 3) == 0) status[1] = t;
        return;
    }
    TC* dst = keys + static_cast<size_t>(page) * key_page_stride + static_cast<size_t>(pos % page_size) * (R + P);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) { const float a = row[dkv_off + i]; ss += a * a; }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(R) + eps);
    for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_f32<TC>(row[dkv_off + i] * inv * wkv[i]);
    const float* kr = row + dkv_off + R;
    const int half = dims / 2;
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
        float v = kr[i];
        if (i < dims) {
            const int f = i < half ? i : i - half;
            float sn, cs;
            sincosf(static_cast<float>(pos) * inv_freq[f], &sn, &cs);
            v = i < half ? kr[i] * cs - kr[i + half] * sn : kr[i] * cs + kr[i - half] * sn;
        }
        dst[R + i] = from_f32<TC>(v);
    }
}

extern "C" int llm_latent_prepare(
    const float* proj, long long proj_stride, int dq_off, int dkv_off, int Q, int R, int P, int dims, const float* wq,
    const float* wkv, float eps, const float* inv_freq, void* cq_out, int q_dtype, void* keys, int cache_dtype,
    long long key_page_stride, const int32_t* positions, const int32_t* token_entry, const int32_t* entry_slot,
    const int32_t* block_table, int table_stride, int num_tokens, int page_size, int num_pages, int32_t* status,
    uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (Q <= 0 || R <= 0 || P < 0 || dims < 0 || dims > P || dims % 2) return LLM_REFUSED_SIZE;
    if (keys && (!block_table || page_size <= 0 || !wkv || (dims > 0 && !inv_freq))) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!keys) cache_dtype = q_dtype;
#define LAUNCH(TQ, TC)                                                                                              \
    launch_pdl((latent_prepare_kernel<TQ, TC>), dim3(num_tokens), dim3(LA_THREADS), 0, s, proj, proj_stride, dq_off,  \
               dkv_off, Q, R, P, dims, wq, wkv, eps, inv_freq, static_cast<TQ*>(cq_out), static_cast<TC*>(keys),     \
               key_page_stride, positions, token_entry, entry_slot, block_table, table_stride, page_size, num_pages, \
               status)
    if (q_dtype == LLM_DT_F32 && cache_dtype == LLM_DT_F32) LAUNCH(float, float);
    else if (q_dtype == LLM_DT_BF16 && cache_dtype == LLM_DT_BF16) LAUNCH(bf16, bf16);
    else if (q_dtype == LLM_DT_F32 && cache_dtype == LLM_DT_BF16) LAUNCH(float, bf16);
    else if (q_dtype == LLM_DT_BF16 && cache_dtype == LLM_DT_F32) LAUNCH(bf16, float);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}

// grid (tokens, heads)
template <typename TQ>
__global__ void latent_q_split_kernel(const float* __restrict__ q, TQ* __restrict__ qn, TQ* __restrict__ packed,
                                      const int32_t* __restrict__ positions, const float* __restrict__ inv_freq,
                                      int num_tokens, int H, int D, int P, int R, int dims) {
    pdl_begin();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* src = q + (static_cast<size_t>(t) * H + h) * (D + P);
    TQ* n = qn + (static_cast<size_t>(h) * num_tokens + t) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) n[i] = from_f32<TQ>(src[i]);
    TQ* dst = packed + (static_cast<size_t>(t) * H + h) * (R + P) + R;
    const float* qr = src + D;
    const int half = dims / 2;
    const float pos = static_cast<float>(positions[t]);
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
        float v = qr[i];
        if (i < dims) {
            const int f = i < half ? i : i - half;
            float sn, cs;
            sincosf(pos * inv_freq[f], &sn, &cs);
            v = i < half ? qr[i] * cs - qr[i + half] * sn : qr[i] * cs + qr[i - half] * sn;
        }
        dst[i] = from_f32<TQ>(v);
    }
}

extern "C" int llm_latent_q_split(const float* q, void* qn, void* packed, int dtype, const int32_t* positions,
                                  const float* inv_freq, int num_tokens, int H, int D, int P, int R, int dims,
                                  uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (H <= 0 || H > 65535 || D <= 0 || P < 0 || R <= 0 || dims < 0 || dims > P || dims % 2 || (dims > 0 && !inv_freq))
        return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int threads = (D > 64 || P > 64) ? 128 : 64;
    if (dtype == LLM_DT_F32)
        launch_pdl((latent_q_split_kernel<float>), dim3(num_tokens, H), dim3(threads), 0, s, q, static_cast<float*>(qn),
                   static_cast<float*>(packed), positions, inv_freq, num_tokens, H, D, P, R, dims);
    else if (dtype == LLM_DT_BF16)
        launch_pdl((latent_q_split_kernel<bf16>), dim3(num_tokens, H), dim3(threads), 0, s, q, static_cast<bf16*>(qn),
                   static_cast<bf16*>(packed), positions, inv_freq, num_tokens, H, D, P, R, dims);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}
