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
// Rotation: the first `dims` entries of the P-part, entry i paired with i + dims/2 (`rot_pairs` 0) or entry 2i with
// 2i + 1 (1), by the angle float(position) * inv_freq[i], sine and cosine in 32-bit and both times `rot_mag`; the
// rest passes unchanged.  Norms are 32-bit.
#include "common.cuh"
#include <math_constants.h>

#define LA_THREADS 256

// entry i (< dims) of a rotated part x at position pos
__device__ __forceinline__ float la_rotated(const float* x, int i, int dims, float pos, const float* inv_freq,
                                            int rot_pairs, float rot_mag) {
    const int half = dims / 2;
    const bool first = rot_pairs ? (i & 1) == 0 : i < half;
    const int f = rot_pairs ? i >> 1 : (first ? i : i - half);
    const int other = rot_pairs ? (i ^ 1) : (first ? i + half : i - half);
    float sn, cs;
    sincosf(pos * inv_freq[f], &sn, &cs);
    return (first ? x[i] * cs - x[other] * sn : x[i] * cs + x[other] * sn) * rot_mag;
}

template <typename TQ, typename TC>
__global__ void latent_prepare_kernel(
    const float* __restrict__ proj, long long proj_stride, int dq_off, int dkv_off, int Q, int R, int P, int dims,
    const float* __restrict__ wq, const float* __restrict__ wkv, float eps, const float* __restrict__ inv_freq,
    TQ* __restrict__ cq_out, TC* __restrict__ keys, long long key_page_stride,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_entry,
    const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table, int table_stride,
    int page_size, int num_pages, int32_t* __restrict__ status, int rot_pairs, float rot_mag) {
    pdl_begin();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float* row = proj + static_cast<size_t>(t) * proj_stride;
    // the page lookup and both latents' loads are started before anything waits: the kernel is bound by their latency
    int pos = 0, page = -1;
    if (keys) {
        pos = positions[t];
        const int slot = entry_slot[token_entry[t]];
        const int logical = pos / page_size;
        page = logical < table_stride ? block_table[static_cast<size_t>(slot) * table_stride + logical] : -1;
    }
    float ss = 0.0f, ss_kv = 0.0f;
    for (int i = threadIdx.x; i < Q; i += blockDim.x) { const float a = row[dq_off + i]; ss += a * a; }
    if (keys)
        for (int i = threadIdx.x; i < R; i += blockDim.x) { const float a = row[dkv_off + i]; ss_kv += a * a; }
    {
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(Q) + eps);
        for (int i = threadIdx.x; i < Q; i += blockDim.x)
            cq_out[static_cast<size_t>(t) * Q + i] = from_f32<TQ>(row[dq_off + i] * inv * wq[i]);
    }
    if (!keys) return;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && atomicCAS(status, 0, 3) == 0) status[1] = t;
        return;
    }
    TC* dst = keys + static_cast<size_t>(page) * key_page_stride + static_cast<size_t>(pos % page_size) * (R + P);
    const float inv = 1.0f / sqrtf(block_sum(ss_kv, scratch) / static_cast<float>(R) + eps);
    for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_f32<TC>(row[dkv_off + i] * inv * wkv[i]);
    const float* kr = row + dkv_off + R;
    for (int i = threadIdx.x; i < P; i += blockDim.x)
        dst[R + i] = from_f32<TC>(i < dims ? la_rotated(kr, i, dims, static_cast<float>(pos), inv_freq, rot_pairs, rot_mag) : kr[i]);
}

extern "C" int llm_latent_prepare(
    const float* proj, long long proj_stride, int dq_off, int dkv_off, int Q, int R, int P, int dims, const float* wq,
    const float* wkv, float eps, const float* inv_freq, void* cq_out, int q_dtype, void* keys, int cache_dtype,
    long long key_page_stride, const int32_t* positions, const int32_t* token_entry, const int32_t* entry_slot,
    const int32_t* block_table, int table_stride, int num_tokens, int page_size, int num_pages, int32_t* status,
    int rot_pairs, float rot_mag, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (Q <= 0 || R <= 0 || P < 0 || dims < 0 || dims > P || dims % 2) return LLM_REFUSED_SIZE;
    if (keys && (!block_table || page_size <= 0 || !wkv || (dims > 0 && !inv_freq))) return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!keys) cache_dtype = q_dtype;
#define LAUNCH(TQ, TC)                                                                                              \
    launch_pdl((latent_prepare_kernel<TQ, TC>), dim3(num_tokens), dim3(LA_THREADS), 0, s, proj, proj_stride, dq_off,  \
               dkv_off, Q, R, P, dims, wq, wkv, eps, inv_freq, static_cast<TQ*>(cq_out), static_cast<TC*>(keys),     \
               key_page_stride, positions, token_entry, entry_slot, block_table, table_stride, page_size, num_pages, \
               status, rot_pairs, rot_mag)
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
                                      int num_tokens, int H, int D, int P, int R, int dims, int rot_pairs, float rot_mag) {
    pdl_begin();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* src = q + (static_cast<size_t>(t) * H + h) * (D + P);
    TQ* n = qn + (static_cast<size_t>(h) * num_tokens + t) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) n[i] = from_f32<TQ>(src[i]);
    TQ* dst = packed + (static_cast<size_t>(t) * H + h) * (R + P) + R;
    const float* qr = src + D;
    const float pos = static_cast<float>(positions[t]);
    for (int i = threadIdx.x; i < P; i += blockDim.x)
        dst[i] = from_f32<TQ>(i < dims ? la_rotated(qr, i, dims, pos, inv_freq, rot_pairs, rot_mag) : qr[i]);
}

extern "C" int llm_latent_q_split(const float* q, void* qn, void* packed, int dtype, const int32_t* positions,
                                  const float* inv_freq, int num_tokens, int H, int D, int P, int R, int dims,
                                  int rot_pairs, float rot_mag, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    if (H <= 0 || H > 65535 || D <= 0 || P < 0 || R <= 0 || dims < 0 || dims > P || dims % 2 || (dims > 0 && !inv_freq))
        return LLM_REFUSED_SIZE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int threads = (D > 64 || P > 64) ? 128 : 64;
    if (dtype == LLM_DT_F32)
        launch_pdl((latent_q_split_kernel<float>), dim3(num_tokens, H), dim3(threads), 0, s, q, static_cast<float*>(qn),
                   static_cast<float*>(packed), positions, inv_freq, num_tokens, H, D, P, R, dims, rot_pairs, rot_mag);
    else if (dtype == LLM_DT_BF16)
        launch_pdl((latent_q_split_kernel<bf16>), dim3(num_tokens, H), dim3(threads), 0, s, q, static_cast<bf16*>(qn),
                   static_cast<bf16*>(packed), positions, inv_freq, num_tokens, H, D, P, R, dims, rot_pairs, rot_mag);
    else
        return LLM_REFUSED_DTYPE;
    return launch_status();
}

// ---- attention over the cached rows on the tensor cores (bfloat16) --------------------------------------------
// One CTA per (token, block of up to 32 heads, split of the token's rows): all heads of a token read the same rows,
// so a tile of 64 rows [c | kr] is staged once in shared memory (cp.async, two buffers, one page lookup per row) and
// serves the scores of every head AND, through its first R entries, their values.  Eight warps per group of 16 heads
// (one group when the layer has at most 16 heads, else two: 256 or 512 threads).  Per tile each of a group's eight
// warps scores 8 of the 64 rows against the packed query [q_abs | q_rot] (mma.sync m16n8k16 over R + P, four
// accumulator chains), the eight exchange row maxima through shared memory (a named barrier per group), write their
// weights as bfloat16, and then each adds weights x rows for its eighth of the R value entries (accumulators in
// registers: R / 64 tiles of 16 x 8) and sums the weights it read, as rounded.  Softmax runs in the exp2 domain, in
// 32-bit, with a running maximum.  A token's window is walked from its first visible row, so every tile holds a
// visible row and the maxima stay finite; rows of a tile beyond the token's position are zero-filled and masked.
// Few tokens (decoding): the tiles of a token are dealt to `splits` CTAs, each leaves its unnormalised sums with its
// maximum and weight sum in float32, and a second kernel merges them.  Prompt portions and single decoded tokens take
// the same path: what a CTA does depends on the token's position only.  R in {64, 128, 256, 512}, R + P a multiple
// of 16, as wide as two buffers of rows and the queries fit in shared memory (R + P up to 704).
#define LM_GROUP_THREADS 256         // eight warps work for 16 heads
#define LM_KEYS 64
#define LM_PS_LD 72                    // a row of weights: 64 and a pad
#define LM_MAX_SPLITS 16

__device__ __forceinline__ void lm_ldsm4(unsigned (&r)[4], const void* p) {
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_ldsm4_t(unsigned (&r)[4], const void* p) {
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lm_cp16(void* dst, const void* src) {
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(src));
}
__device__ __forceinline__ void lm_group_sync(int group) {          // the eight warps of a group of heads
    asm volatile("bar.sync %0, 256;\n" ::"r"(group + 1) : "memory");
}
__device__ __forceinline__ float lm_pair_sum(unsigned u) {          // two bfloat16 in a register, summed
    return __uint_as_float(u << 16) + __uint_as_float(u & 0xffff0000u);
}

template <int NT>   // NT = R / 64: value tiles of 8 entries a warp accumulates
__global__ void __launch_bounds__(2 * LM_GROUP_THREADS) latent_attention_mma_kernel(
    const bf16* __restrict__ q, bf16* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml,
    const bf16* __restrict__ rows_cache, long long page_stride, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ token_entry, const int32_t* __restrict__ entry_slot, const int32_t* __restrict__ block_table,
    int table_stride, int H, int DK, int page_size, int window, float scale_log2e, int num_pages,
    int32_t* __restrict__ status) {
    pdl_begin();
    constexpr int R = NT * 64, STAGES = 2;
    extern __shared__ __align__(16) unsigned char lm_smem[];
    const int ld = DK + 8;                                               // padded row: ldmatrix without bank conflicts
    const int groups = blockDim.x / LM_GROUP_THREADS, block_heads = 16 * groups, nwarps = blockDim.x >> 5;
    bf16* qs = reinterpret_cast<bf16*>(lm_smem);                          // [16 per group][ld]
    bf16* ks = qs + block_heads * ld;                                     // [2][64 rows][ld]
    bf16* ps = ks + STAGES * LM_KEYS * ld;                                // [groups][16][72] weights of the tile
    float* red = reinterpret_cast<float*>(ps + groups * 16 * LM_PS_LD);   // [groups][8 warps][16 rows] maxima
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rg = warp >> 3, eighth = warp & 7, g = lane >> 2, c = lane & 3;
    const int t = blockIdx.x, h0 = blockIdx.y * block_heads, splits = gridDim.z, z = blockIdx.z;
    const int heads_here = min(block_heads, H - h0);
    const int pos = positions[t];
    const int slot = entry_slot[token_entry[t]];
    const int32_t* table = block_table + static_cast<size_t>(slot) * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int chunks = DK / 8;                                           // 16-byte pieces of a row
    const int n_tiles = (pos - lo) / LM_KEYS + 1;
    const int per = (n_tiles + splits - 1) / splits;
    const int first = z * per, last = min(first + per, n_tiles);        // this CTA's tiles; tile i starts at row lo + 64 i
    const bool active = rg * 16 < heads_here;                            // a row group without heads only keeps the barriers
    const int r0 = rg * 16 + g, r1 = r0 + 8;

    if (first >= last) {                                                 // more splits than tiles: nothing to add
        if (active && eighth == 0 && c == 0) {
            float* ml = part_ml + (static_cast<size_t>(t) * splits + z) * H * 2;
            if (r0 < heads_here) { ml[(h0 + r0) * 2] = -CUDART_INF_F; ml[(h0 + r0) * 2 + 1] = 0.0f; }
            if (r1 < heads_here) { ml[(h0 + r1) * 2] = -CUDART_INF_F; ml[(h0 + r1) * 2 + 1] = 0.0f; }
        }
        return;
    }

    auto stage = [&](int tile, int buf) {                                // a warp brings whole rows
        bf16* dst = ks + static_cast<size_t>(buf) * LM_KEYS * ld;
        const int kt = lo + tile * LM_KEYS;
        for (int r = warp; r < LM_KEYS; r += nwarps) {
            const int j = kt + r;
            const bf16* src = nullptr;
            if (j <= pos) {
                const int logical = j / page_size;
                const int page = logical < table_stride ? table[logical] : -1;
                if (page < 0 || page >= num_pages) {
                    if (lane == 0 && atomicCAS(status, 0, 4) == 0) status[1] = t;
                } else {
                    src = rows_cache + static_cast<long long>(page) * page_stride + static_cast<size_t>(j - logical * page_size) * DK;
                }
            }
            bf16* d = dst + r * ld;
            if (src) {
                for (int ch = lane; ch < chunks; ch += 32) lm_cp16(d + ch * 8, src + ch * 8);
            } else {
                for (int ch = lane; ch < chunks; ch += 32) *reinterpret_cast<uint4*>(d + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    auto commit = [] { asm volatile("cp.async.commit_group;\n" ::: "memory"); };

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (first + s < last) stage(first + s, s);
        commit();
    }
    for (int i = tid; i < block_heads * chunks; i += blockDim.x) {          // the packed queries of this block's heads
        const int r = i / chunks, ch = i - r * chunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < heads_here) v = *reinterpret_cast<const uint4*>(q + (static_cast<size_t>(t) * H + h0 + r) * DK + ch * 8);
        *reinterpret_cast<uint4*>(qs + r * ld + ch * 8) = v;
    }
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.0f, l1 = 0.0f;
    bf16* pg = ps + rg * 16 * LM_PS_LD;
    float* redg = red + rg * 8 * 16;
    const bf16* qa = qs + (rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + (lane >> 4) * 8;
    const int frag_row = (lane & 7) + ((lane >> 3) & 1) * 8, frag_col = (lane >> 4) * 8;

    for (int i = first; i < last; ++i) {
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();                             // tile i has landed; the buffer of tile i - 1 is free, its weights read
        if (i + STAGES - 1 < last) stage(i + STAGES - 1, (i + STAGES - 1 - first) % STAGES);
        commit();
        if (!active) continue;
        const int kt = lo + i * LM_KEYS;
        const bf16* kb = ks + static_cast<size_t>((i - first) % STAGES) * LM_KEYS * ld;
        // scores of this warp's 8 rows of the tile, for the group's 16 heads
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s1[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s2[4] = {0.0f, 0.0f, 0.0f, 0.0f},
              s3[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const bf16* kk = kb + (eighth * 8 + (lane & 7)) * ld + (lane >> 3) * 8;
        int k0 = 0;
        for (; k0 + 64 <= DK; k0 += 64) {
            unsigned a[4], a1[4], a2[4], a3[4], b[4], b1[4];
            lm_ldsm4(b, kk + k0);                                        // dims k0 .. k0 + 31 of the 8 rows
            lm_ldsm4(b1, kk + k0 + 32);
            lm_ldsm4(a, qa + k0);
            lm_ldsm4(a1, qa + k0 + 16);
            lm_ldsm4(a2, qa + k0 + 32);
            lm_ldsm4(a3, qa + k0 + 48);
            lm_mma(s, a, b[0], b[1]);
            lm_mma(s1, a1, b[2], b[3]);
            lm_mma(s2, a2, b1[0], b1[1]);
            lm_mma(s3, a3, b1[2], b1[3]);
        }
        for (; k0 < DK; k0 += 16) {                                      // up to three steps of 16 (the upper half of b unused)
            unsigned a[4], b[4];
            lm_ldsm4(b, kk + k0);
            lm_ldsm4(a, qa + k0);
            lm_mma(s, a, b[0], b[1]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) s[u] += s1[u] + (s2[u] + s3[u]);
        const int key = kt + eighth * 8 + 2 * c;
        const bool v0 = key <= pos, v1 = key + 1 <= pos;
        s[0] = v0 ? s[0] * scale_log2e : -CUDART_INF_F;
        s[1] = v1 ? s[1] * scale_log2e : -CUDART_INF_F;
        s[2] = v0 ? s[2] * scale_log2e : -CUDART_INF_F;
        s[3] = v1 ? s[3] * scale_log2e : -CUDART_INF_F;
        float x0 = fmaxf(s[0], s[1]), x1 = fmaxf(s[2], s[3]);
        x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 1));
        x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 2));
        x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 1));
        x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 2));
        if (c == 0) {
            redg[eighth * 16 + g] = x0;
            redg[eighth * 16 + g + 8] = x1;
        }
        lm_group_sync(rg);
        float t0 = redg[g], t1 = redg[g + 8];
#pragma unroll
        for (int w2 = 1; w2 < 8; ++w2) {
            t0 = fmaxf(t0, redg[w2 * 16 + g]);
            t1 = fmaxf(t1, redg[w2 * 16 + g + 8]);
        }
        const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);             // finite: the tile's first row is visible
        const float al0 = (m0 == -CUDART_INF_F) ? 0.0f : exp2f(m0 - n0);
        const float al1 = (m1 == -CUDART_INF_F) ? 0.0f : exp2f(m1 - n1);
        m0 = n0;
        m1 = n1;
        // the weights as the value product will read them: rounded to bfloat16 (and summed as rounded, below)
        *reinterpret_cast<__nv_bfloat162*>(pg + g * LM_PS_LD + eighth * 8 + 2 * c) = __floats2bfloat162_rn(exp2f(s[0] - n0), exp2f(s[1] - n0));
        *reinterpret_cast<__nv_bfloat162*>(pg + (g + 8) * LM_PS_LD + eighth * 8 + 2 * c) = __floats2bfloat162_rn(exp2f(s[2] - n1), exp2f(s[3] - n1));
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            acc[n][0] *= al0;
            acc[n][1] *= al0;
            acc[n][2] *= al1;
            acc[n][3] *= al1;
        }
        lm_group_sync(rg);
        // weights [16 x 64] times the rows' first R entries, this warp's eighth of them
        unsigned pa[4][4];
        float u0 = 0.0f, u1 = 0.0f;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
            lm_ldsm4(pa[k4], pg + frag_row * LM_PS_LD + k4 * 16 + frag_col);
            u0 += lm_pair_sum(pa[k4][0]) + lm_pair_sum(pa[k4][2]);
            u1 += lm_pair_sum(pa[k4][1]) + lm_pair_sum(pa[k4][3]);
        }
        u0 += __shfl_xor_sync(0xffffffffu, u0, 1);
        u0 += __shfl_xor_sync(0xffffffffu, u0, 2);
        u1 += __shfl_xor_sync(0xffffffffu, u1, 1);
        u1 += __shfl_xor_sync(0xffffffffu, u1, 2);
        l0 = l0 * al0 + u0;
        l1 = l1 * al1 + u1;
        const bf16* vb = kb + frag_row * ld + eighth * (R / 8) + frag_col;
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {                             // rows 16 k4 .. 16 k4 + 15 of the tile
                unsigned b[4];
                lm_ldsm4_t(b, vb + k4 * 16 * ld + n * 8);
                lm_mma(acc[n], pa[k4], b[0], b[1]);
                if (n + 1 < NT) lm_mma(acc[n + 1 < NT ? n + 1 : n], pa[k4], b[2], b[3]);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    if (!active) return;
    if (splits == 1) {
        const float i0 = 1.0f / l0, i1 = 1.0f / l1;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int col = eighth * (R / 8) + n * 8 + 2 * c;
            if (r0 < heads_here)
                *reinterpret_cast<__nv_bfloat162*>(out + (static_cast<size_t>(t) * H + h0 + r0) * R + col) =
                    __floats2bfloat162_rn(acc[n][0] * i0, acc[n][1] * i0);
            if (r1 < heads_here)
                *reinterpret_cast<__nv_bfloat162*>(out + (static_cast<size_t>(t) * H + h0 + r1) * R + col) =
                    __floats2bfloat162_rn(acc[n][2] * i1, acc[n][3] * i1);
        }
        return;
    }
    const size_t base = (static_cast<size_t>(t) * splits + z) * H;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const int col = eighth * (R / 8) + n * 8 + 2 * c;
        if (r0 < heads_here) *reinterpret_cast<float2*>(part_acc + (base + h0 + r0) * R + col) = make_float2(acc[n][0], acc[n][1]);
        if (r1 < heads_here) *reinterpret_cast<float2*>(part_acc + (base + h0 + r1) * R + col) = make_float2(acc[n][2], acc[n][3]);
    }
    if (eighth == 0 && c == 0) {
        if (r0 < heads_here) { part_ml[(base + h0 + r0) * 2] = m0; part_ml[(base + h0 + r0) * 2 + 1] = l0; }
        if (r1 < heads_here) { part_ml[(base + h0 + r1) * 2] = m1; part_ml[(base + h0 + r1) * 2 + 1] = l1; }
    }
}

// out[t, h, :] = sum_z 2^(m_z - M) acc_z / sum_z 2^(m_z - M) l_z over the splits of (t, h); M the largest m_z.
// One warp a (token, head); the loops run over all LM_MAX_SPLITS with a predicate, so that the loads of the splits
// are in flight together; what an empty split left in `part_acc` is never read.
__global__ void latent_attention_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                              bf16* __restrict__ out, int H, int R, int splits, int pairs) {
    pdl_begin();
    const int lane = threadIdx.x & 31, pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const int t = pair / H, h = pair - t * H;
    const size_t base = static_cast<size_t>(t) * splits * H + h;        // split z sits at base + z * H
    float mz[LM_MAX_SPLITS], M = -CUDART_INF_F, L = 0.0f;
#pragma unroll
    for (int z = 0; z < LM_MAX_SPLITS; ++z) {
        mz[z] = z < splits ? part_ml[(base + static_cast<size_t>(z) * H) * 2] : -CUDART_INF_F;
        M = fmaxf(M, mz[z]);
    }
#pragma unroll
    for (int z = 0; z < LM_MAX_SPLITS; ++z) {
        const float l = z < splits ? part_ml[(base + static_cast<size_t>(z) * H) * 2 + 1] : 0.0f;
        mz[z] = (mz[z] == -CUDART_INF_F) ? 0.0f : exp2f(mz[z] - M);     // from here on: the split's weight
        L += mz[z] * l;
    }
    const float inv = 1.0f / L;
    for (int col = lane * 2; col < R; col += 64) {
        float2 v[LM_MAX_SPLITS];
#pragma unroll
        for (int z = 0; z < LM_MAX_SPLITS; ++z)
            v[z] = mz[z] != 0.0f ? *reinterpret_cast<const float2*>(part_acc + (base + static_cast<size_t>(z) * H) * R + col)
                                 : make_float2(0.0f, 0.0f);
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
        for (int z = 0; z < LM_MAX_SPLITS; ++z) {
            a0 += mz[z] * v[z].x;
            a1 += mz[z] * v[z].y;
        }
        *reinterpret_cast<__nv_bfloat162*>(out + (static_cast<size_t>(t) * H + h) * R + col) = __floats2bfloat162_rn(a0 * inv, a1 * inv);
    }
}

static size_t lm_smem_bytes(int DK, int groups) {
    return static_cast<size_t>(16 * groups + 2 * LM_KEYS) * (DK + 8) * sizeof(bf16) + groups * 16 * LM_PS_LD * sizeof(bf16) +
           groups * 8 * 16 * sizeof(float);
}

extern "C" int llm_latent_attention_supported(int R, int P) {
    return (R == 64 || R == 128 || R == 256 || R == 512) && P >= 0 && (R + P) % 16 == 0 && lm_smem_bytes(R + P, 2) <= 227 * 1024;
}

// Into how many CTAs a token's rows are dealt: one when the tokens alone fill the GPU twice, else enough for that, at
// most one per tile of the longest walk a token of this step can have (its window, or all pages of its table).
extern "C" int llm_latent_attention_splits(int num_tokens, int H, int window, int table_stride, int page_size) {
    const long long ctas = static_cast<long long>(num_tokens) * ((H + 31) / 32);
    if (ctas <= 0 || ctas >= 2 * 148) return 1;
    const long long rows = window > 0 ? window : static_cast<long long>(table_stride) * page_size;
    const long long tiles = (rows + LM_KEYS - 1) / LM_KEYS;
    long long s = (2 * 148 + ctas - 1) / ctas;
    if (s > tiles) s = tiles;
    if (s > LM_MAX_SPLITS) s = LM_MAX_SPLITS;
    return s < 1 ? 1 : static_cast<int>(s);
}

// q: bfloat16 [T, H * (R + P)] packed queries; out: bfloat16 [T, H * R]; rows_cache: bfloat16 [pages, 1, page, R + P];
// splits > 1: part_acc float32 [T, splits, H, R] and part_ml float32 [T, splits, H, 2] are the kernels' scratch.
extern "C" int llm_latent_attention(const void* q, void* out, float* part_acc, float* part_ml, int splits,
                                    const void* rows_cache, long long page_stride, const int32_t* positions,
                                    const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table,
                                    int table_stride, int num_tokens, int H, int R, int P, int page_size, int window,
                                    float scale, int num_pages, int32_t* status, uintptr_t stream) {
    if (num_tokens <= 0) return LLM_OK;
    const int groups = H > 16 ? 2 : 1, blocks = (H + 16 * groups - 1) / (16 * groups);
    if (!llm_latent_attention_supported(R, P) || H <= 0 || page_size <= 0 || blocks > 65535 || splits < 1 ||
        splits > LM_MAX_SPLITS || (splits > 1 && (!part_acc || !part_ml)))
        return LLM_REFUSED_SIZE;
    if (!aligned16(q) || !aligned16(out) || !aligned16(rows_cache) || page_stride % 8 || (part_acc && !aligned16(part_acc)))
        return LLM_REFUSED_ALIGN;
    const int DK = R + P;
    const size_t smem = lm_smem_bytes(DK, groups);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const dim3 grid(num_tokens, blocks, splits);
#define LAUNCH(NT)                                                                                                    \
    {                                                                                                                 \
        auto kern = latent_attention_mma_kernel<NT>;                                                                  \
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                                                   static_cast<int>(smem));                                           \
        if (e != cudaSuccess) return static_cast<int>(e);                                                             \
        launch_pdl(kern, grid, dim3(groups * LM_GROUP_THREADS), smem, s, static_cast<const bf16*>(q),                 \
                   static_cast<bf16*>(out), part_acc, part_ml, static_cast<const bf16*>(rows_cache), page_stride,     \
                   positions, token_entry, entry_slot, block_table, table_stride, H, DK, page_size, window,           \
                   scale * 1.4426950408889634f, num_pages, status);                                                   \
    }
    if (R == 64) LAUNCH(1) else if (R == 128) LAUNCH(2) else if (R == 256) LAUNCH(4) else LAUNCH(8)
#undef LAUNCH
    if (splits > 1)
        launch_pdl(latent_attention_merge_kernel, dim3((num_tokens * H + 3) / 4), dim3(128), 0, s,
                   static_cast<const float*>(part_acc), static_cast<const float*>(part_ml), static_cast<bf16*>(out), H, R, splits,
                   num_tokens * H);
    return launch_status();
}
