// Everything between the q/k/v projection and the attention kernel, for attention layers that are
// not of the "per-head norm, then rotation" kind that `rope_cache.cu` fuses.  One block per token:
//
//   q = proj[t, q_off : q_off + nq*dk] (+ bq)        k = proj[t, k_off : ...] (+ bk)      v likewise (+ bv)
//   norm (32-bit), by `norm_scope`:
//       0  none
//       1  per head:        x_head * rsqrt(mean(x_head^2) + eps) * w[i mod dk]
//       2  whole projection: x * rsqrt(mean over ALL heads' entries of x^2 + eps) * w[i]
//   rotation (optional, after the norm): of the first rot_dims entries of every q and k head, pairs (2i, 2i + 1)
//       (`rot_pairs` 1) or (i, i + rot_dims/2) (0) turn by the angle float(p) * rot_freq[i]; the pair (a, b) becomes
//       (a cos - b sin, b cos + a sin) * rot_mag.  `rot_freq` is a float32 table [rot_dims/2] that its owner makes
//       (any stretching of the frequencies is the owner's); angle, sine and cosine are 32-bit.
//   query temperature (optional): q *= 1 + coef * ln(floor((p + 1) / every) + 1), p the token's position
//   q is stored in the compute dtype [T, nq*dk]; k and v go to the token's place in its request's
//   pages, `keys` [pages, nkv, page, dk] and `values` [pages, nkv, page, dv] (any page strides, so that
//   the two halves of one [pages, 2, nkv, page, d] tensor are served as well as tensors of their own).
//
// `proj` is float32 (the projection's accumulators, never rounded on their way here), `proj_stride`
// floats from token to token: the three pieces may be columns of a wider product.
#include "common.cuh"

#define AP_THREADS 256

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(bf16* p, float4 v) {
    uint2 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
    h[0] = __floats2bfloat162_rn(v.x, v.y);
    h[1] = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ float4 scale4(float4 a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }
__device__ __forceinline__ float sq4(float4 a) { return a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w; }

template <typename TQ, typename TC>
__global__ void attention_prepare_kernel(
    const float* __restrict__ proj, long long proj_stride, int q_off, int k_off, int v_off,
    const float* __restrict__ bq, const float* __restrict__ bk, const float* __restrict__ bv,
    const float* __restrict__ qw, const float* __restrict__ kw, int norm_scope, float eps,
    float temp_coef, int temp_every,
    TQ* __restrict__ q_out, TC* __restrict__ keys, TC* __restrict__ values,
    long long key_page_stride, long long value_page_stride,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table, int table_stride,
    int nq, int nkv, int dk, int dv, int page_size, int num_pages, int vec, int32_t* __restrict__ status,
    const float* __restrict__ rot_freq, int rot_dims, float rot_mag, int rot_pairs) {
    pdl_begin();
    extern __shared__ __align__(16) float smem[];
    const int nqe = nq * dk, nke = nkv * dk, nve = nkv * dv;
    float* fq = smem;                       // [nq*dk]
    float* fk = smem + nqe;                 // [nkv*dk]
    float* scratch = fk + nke;              // 33
    const int t = blockIdx.x;
    const float* row = proj + static_cast<size_t>(t) * proj_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;

    float ssq = 0.0f, ssk = 0.0f;
    if (vec) {                                  // every width and offset a multiple of four floats: 16-byte accesses
        for (int i = threadIdx.x * 4; i < nqe; i += blockDim.x * 4) {
            float4 a = ld4(row + q_off + i);
            if (bq) a = add4(a, ld4(bq + i));
            st4(fq + i, a);
            ssq += sq4(a);
        }
        if (keys)
            for (int i = threadIdx.x * 4; i < nke; i += blockDim.x * 4) {
                float4 a = ld4(row + k_off + i);
                if (bk) a = add4(a, ld4(bk + i));
                st4(fk + i, a);
                ssk += sq4(a);
            }
    } else {
        for (int i = threadIdx.x; i < nqe; i += blockDim.x) {
            const float a = row[q_off + i] + (bq ? bq[i] : 0.0f);
            fq[i] = a;
            ssq += a * a;
        }
        if (keys)
            for (int i = threadIdx.x; i < nke; i += blockDim.x) {
                const float a = row[k_off + i] + (bk ? bk[i] : 0.0f);
                fk[i] = a;
                ssk += a * a;
            }
    }
    if (norm_scope == 2) {
        // each thread scales what it wrote itself, so no barrier stands between the two passes but the sums'
        const float tq = block_sum(ssq, scratch);
        const float iq = 1.0f / sqrtf(tq / static_cast<float>(nqe) + eps);
        if (vec)
            for (int i = threadIdx.x * 4; i < nqe; i += blockDim.x * 4)
                st4(fq + i, qw ? mul4(scale4(ld4(fq + i), iq), ld4(qw + i)) : scale4(ld4(fq + i), iq));
        else
            for (int i = threadIdx.x; i < nqe; i += blockDim.x) fq[i] = fq[i] * iq * (qw ? qw[i] : 1.0f);
        if (keys) {
            const float tk = block_sum(ssk, scratch);
            const float ik = 1.0f / sqrtf(tk / static_cast<float>(nke) + eps);
            if (vec)
                for (int i = threadIdx.x * 4; i < nke; i += blockDim.x * 4)
                    st4(fk + i, kw ? mul4(scale4(ld4(fk + i), ik), ld4(kw + i)) : scale4(ld4(fk + i), ik));
            else
                for (int i = threadIdx.x; i < nke; i += blockDim.x) fk[i] = fk[i] * ik * (kw ? kw[i] : 1.0f);
        }
    } else if (norm_scope == 1) {
        __syncthreads();
        for (int head = warp; head < nq + (keys ? nkv : 0); head += nwarps) {      // a warp per head
            float* x = head < nq ? fq + head * dk : fk + (head - nq) * dk;
            const float* w = head < nq ? qw : kw;
            float ss = 0.0f;
            for (int i = lane; i < dk; i += 32) ss += x[i] * x[i];
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / static_cast<float>(dk) + eps);
            for (int i = lane; i < dk; i += 32) x[i] = x[i] * inv * (w ? w[i] : 1.0f);
        }
    }
    __syncthreads();

    const int pos = positions[t];
    if (rot_freq) {                             // a thread a pair, over the heads of q and then of k
        const int half = rot_dims >> 1;
        const int pairs = (nq + (keys ? nkv : 0)) * half;
        for (int idx = threadIdx.x; idx < pairs; idx += blockDim.x) {
            const int head = idx / half, i = idx - head * half;
            float* x = head < nq ? fq + head * dk : fk + (head - nq) * dk;
            const int ia = rot_pairs ? 2 * i : i, ib = rot_pairs ? 2 * i + 1 : i + half;
            float sn, cs;
            sincosf(static_cast<float>(pos) * rot_freq[i], &sn, &cs);
            sn *= rot_mag;
            cs *= rot_mag;
            const float a = x[ia], b = x[ib];
            x[ia] = a * cs - b * sn;
            x[ib] = b * cs + a * sn;
        }
        __syncthreads();
    }
    float temp = 1.0f;
    if (temp_every > 0) temp = 1.0f + temp_coef * logf(static_cast<float>((pos + 1) / temp_every + 1));
    TQ* qo = q_out + static_cast<size_t>(t) * nqe;
    if (vec)
        for (int i = threadIdx.x * 4; i < nqe; i += blockDim.x * 4) st4(qo + i, scale4(ld4(fq + i), temp));
    else
        for (int i = threadIdx.x; i < nqe; i += blockDim.x) qo[i] = from_f32<TQ>(fq[i] * temp);
    if (!keys) return;

    const int slot = entry_slot[token_entry[t]];
    const int logical = pos / page_size;
    const int page = logical < table_stride ? block_table[static_cast<size_t>(slot) * table_stride + logical] : -1;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && atomicCAS(status, 0, 3) == 0) status[1] = t;
        return;
    }
    const int in_page = pos % page_size;
    TC* kp = keys + static_cast<size_t>(page) * key_page_stride;
    TC* vp = values + static_cast<size_t>(page) * value_page_stride;
    if (vec) {
        for (int i = threadIdx.x * 4; i < nke; i += blockDim.x * 4) {
            const int head = i / dk, e = i - head * dk;
            st4(kp + (static_cast<size_t>(head) * page_size + in_page) * dk + e, ld4(fk + i));
        }
        for (int i = threadIdx.x * 4; i < nve; i += blockDim.x * 4) {
            const int head = i / dv, e = i - head * dv;
            float4 a = ld4(row + v_off + i);
            if (bv) a = add4(a, ld4(bv + i));
            st4(vp + (static_cast<size_t>(head) * page_size + in_page) * dv + e, a);
        }
        return;
    }
    for (int i = threadIdx.x; i < nke; i += blockDim.x) {
        const int head = i / dk, e = i - head * dk;
        kp[(static_cast<size_t>(head) * page_size + in_page) * dk + e] = from_f32<TC>(fk[i]);
    }
    for (int i = threadIdx.x; i < nve; i += blockDim.x) {
        const int head = i / dv, e = i - head * dv;
        vp[(static_cast<size_t>(head) * page_size + in_page) * dv + e] =
            from_f32<TC>(row[v_off + i] + (bv ? bv[i] : 0.0f));
    }
}

extern "C" int llm_attention_prepare(
    const float* proj, long long proj_stride, int q_off, int k_off, int v_off, const float* bq, const float* bk,
    const float* bv, const float* qw, const float* kw, int norm_scope, float eps, float temp_coef, int temp_every,
    void* q_out, int q_dtype, void* keys, void* values, int cache_dtype, long long key_page_stride,
    long long value_page_stride, const int32_t* positions, const int32_t* token_entry, const int32_t* entry_slot,
    const int32_t* block_table, int table_stride, int num_tokens, int nq, int nkv, int dk, int dv, int page_size,
    int num_pages, int32_t* status, const float* rot_freq, int rot_dims, float rot_mag, int rot_pairs, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (nq <= 0 || nkv < 0 || dk <= 0 || dv <= 0 || norm_scope < 0 || norm_scope > 2 || temp_every < 0)
        return LLM_REFUSED_SIZE;
    if (rot_freq && (rot_dims <= 0 || rot_dims % 2 || rot_dims > dk)) return LLM_REFUSED_SIZE;
    if (keys && (!values || !block_table || page_size <= 0)) return LLM_REFUSED_SIZE;
    const size_t smem = (static_cast<size_t>(nq) * dk + static_cast<size_t>(nkv) * dk + 33) * sizeof(float);
    if (smem > 200 * 1024) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!keys) cache_dtype = q_dtype;
    const bool fours = dk % 4 == 0 && dv % 4 == 0 && proj_stride % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 &&
                       v_off % 4 == 0 && key_page_stride % 4 == 0 && value_page_stride % 4 == 0;
    const int vec = fours && aligned16(proj) && aligned16(q_out) && (!keys || (aligned16(keys) && aligned16(values))) &&
                    (!bq || aligned16(bq)) && (!bk || aligned16(bk)) && (!bv || aligned16(bv)) &&
                    (!qw || aligned16(qw)) && (!kw || aligned16(kw));
#define LAUNCH(TQ, TC)                                                                                            \
    do {                                                                                                          \
        auto kern = attention_prepare_kernel<TQ, TC>;                                                             \
        if (smem > 48 * 1024) {                                                                                   \
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                                       static_cast<int>(smem));                                   \
            if (e != cudaSuccess) return static_cast<int>(e);                                                     \
        }                                                                                                         \
        launch_pdl(kern, dim3(num_tokens), dim3(AP_THREADS), smem, s, proj, proj_stride, q_off, k_off, v_off, bq, \
                   bk, bv, qw, kw, norm_scope, eps, temp_coef, temp_every, static_cast<TQ*>(q_out),               \
                   static_cast<TC*>(keys), static_cast<TC*>(values), key_page_stride, value_page_stride,          \
                   positions, token_entry, entry_slot, block_table, table_stride, nq, nkv, dk, dv, page_size,     \
                   num_pages, vec, status, rot_freq, rot_dims, rot_mag, rot_pairs);                               \
    } while (0)
    if (q_dtype == LLM_DT_F32 && cache_dtype == LLM_DT_F32) LAUNCH(float, float);
    else if (q_dtype == LLM_DT_BF16 && cache_dtype == LLM_DT_BF16) LAUNCH(bf16, bf16);
    else if (q_dtype == LLM_DT_F32 && cache_dtype == LLM_DT_BF16) LAUNCH(float, bf16);
    else if (q_dtype == LLM_DT_BF16 && cache_dtype == LLM_DT_F32) LAUNCH(bf16, float);
    else return LLM_REFUSED_DTYPE;
#undef LAUNCH
    return launch_status();
}

// out[t, out_off + i] = a[t, i] * gate(g[t, g_off + i]) * scale for i < width, in 32-bit, stored in the
// compute dtype: the output gate of an attention layer whose attention ran in a kernel that knows no
// gate.  gate_kind 0: none (scale and place only), 1: sigmoid, 2: silu.  `a` is contiguous [T, width]; g is float32 with `g_stride`
// floats a row, out has `out_stride` elements a row.
template <typename T>
__global__ void gate_mul_kernel(const T* __restrict__ a, const float* __restrict__ g, long long g_stride, int g_off,
                                T* __restrict__ out, long long out_stride, int out_off, int width, int gate_kind,
                                float scale, int vec, int per_head) {
    // per_head > 0: one gate value per head of `per_head` channels (gate column g_off + channel / per_head)
    pdl_begin();
    const size_t t = blockIdx.y;
    if (vec) {                                       // 16-byte accesses, 8 elements a thread a trip
        for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8; i < width; i += gridDim.x * blockDim.x * 8) {
            float x[8], z[8];
            load8(a + t * width + i, x);
            if (gate_kind != 0) {
                if (per_head > 0) {                  // eight neighbours share a head (per_head is a multiple of 8 here)
                    const float one = g[t * g_stride + g_off + i / per_head];
#pragma unroll
                    for (int u = 0; u < 8; ++u) z[u] = one;
                } else {
                    load8(g + t * g_stride + g_off + i, z);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const float s = 1.0f / (1.0f + expf(-z[u]));
                    x[u] *= (gate_kind == 2 ? z[u] * s : s);
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] *= scale;
            store8(out + t * out_stride + out_off + i, x);
        }
        return;
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < width; i += gridDim.x * blockDim.x) {
        float gate = 1.0f;
        if (gate_kind != 0) {
            const float z = g[t * g_stride + g_off + (per_head > 0 ? i / per_head : i)];
            const float s = 1.0f / (1.0f + expf(-z));
            gate = gate_kind == 2 ? z * s : s;
        }
        out[t * out_stride + out_off + i] = from_f32<T>(to_f32(a[t * width + i]) * gate * scale);
    }
}

extern "C" int llm_gate_mul(const void* a, int dtype, const float* g, long long g_stride, int g_off, void* out,
                            long long out_stride, int out_off, int num_tokens, int width, int gate_kind, float scale,
                            int per_head, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (width <= 0 || num_tokens > 65535 || gate_kind < 0 || gate_kind > 2 || (gate_kind && !g)) return LLM_REFUSED_SIZE;
    const int threads = 256;
    const int esz = dtype == LLM_DT_F32 ? 4 : 2;
    if (per_head < 0) return LLM_REFUSED_SIZE;
    // sixteen-byte accesses: per channel the gate row is read in eights too; per head eight neighbours share one value
    const int vec = width % 8 == 0 && out_stride % 8 == 0 && out_off % 8 == 0 && aligned16(a) && aligned16(out) && esz > 0 &&
                    (per_head > 0 ? per_head % 8 == 0 : (!g || (aligned16(g) && g_stride % 4 == 0 && g_off % 4 == 0)));
    const int per_row = vec ? width / 8 : width;
    const int bx = (per_row + threads - 1) / threads;
    const dim3 grid(bx < 64 ? bx : 64, num_tokens);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == LLM_DT_F32)
        launch_pdl((gate_mul_kernel<float>), grid, dim3(threads), 0, s, static_cast<const float*>(a), g, g_stride, g_off,
                   static_cast<float*>(out), out_stride, out_off, width, gate_kind, scale, vec, per_head);
    else if (dtype == LLM_DT_BF16)
        launch_pdl((gate_mul_kernel<bf16>), grid, dim3(threads), 0, s, static_cast<const bf16*>(a), g, g_stride, g_off,
                   static_cast<bf16*>(out), out_stride, out_off, width, gate_kind, scale, vec, per_head);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}
