// Latent attention: every head's keys and values are projections of one small latent per
// token, so the cache keeps, per token, the record [c (kv_rank) | kr (rot_dim)]: the normed
// latent and a rotated key slice that is the same for every head.  With the up-projections folded into
// the query and the output,
//     score_h(i, j) = (q'_h(i) . c_j + rot(qr_h(i)) . kr_j) * scale,   q'_h = W_uk_h^T q_nope_h,
//     o_h(i) = W_uv_h (sum_j p_h(i, j) c_j),
// attention is one key/value "head" of width kv_rank + rot_dim (values: the first kv_rank)
// that all query heads read.  This file holds the mechanism's plain kernels, for both
// element types and every size:
//   latent_prep          per token: RMSNorm of c with its weight, rotation of kr and of the
//                        heads' rotated query parts (neighbouring pairs (2i, 2i+1), angle
//                        pos * inv_freq[i]), the record into the paged pool
//   head_linear          out[t, h, :] = W[h] x[t, h, :] for per-head matrices (folding W_uk
//                        into the query, W_uv out of the attention's output)
//   latent_attention     softmax attention of packed query tokens over the paged records;
//                        sums in an order that depends only on the query's own position
// Everything the arithmetic touches is fp32; the element type is that of storage.
#include "common.cuh"

// ---------------------------------------------------------------------------- prep
// One block per token.  q [T, H, dn + dr] and dkv [T, r + dr] are views of the fused projection's rows
// (dkv is absent for a layer that reads another layer's records).  rec_out (may be null): the token's record also goes
// to row t of a plain matrix [T, r + dr], for a step that multiplies its own records at once.
template <typename TA>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const TA* q, int q_stride, TA* qo, int qo_stride, int qo_hstride,
                   const TA* __restrict__ dkv, int dkv_stride, VecW cw, float eps,
                   const float* __restrict__ inv_freq, int n_rot, const int* __restrict__ token_pos,
                   const int* __restrict__ token_slot, const int* __restrict__ block_table, int table_stride,
                   TA* __restrict__ pool, int H, int dn, int dr, int r, TA* __restrict__ rec_out, int rec_stride) {
    __shared__ float red[32];
    __shared__ float cs[2][256];               // cos, sin of the token's angles
    pdl_trigger();
    const int t = blockIdx.x;
    if (!ZLM_CHK(token_pos + t, 4)) return;
    const int pos = token_pos[t];
    const int ang = n_rot / 2;
    for (int i = threadIdx.x; i < ang; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[0][i] = c;
        cs[1][i] = s;
    }
    pdl_wait();
    __syncthreads();
    // the heads' rotated query parts: from q[t, h, dn:] to qo[t, h, :dr] (which may be the same place)
    const TA* qr = q + (size_t)t * q_stride;
    TA* qw = qo + (size_t)t * qo_stride;
    const int half = dr / 2 + (dr & 1);         // pairs, and a last single one if dr is odd
    for (int e = threadIdx.x; e < H * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        const TA* p = qr + (size_t)h * (dn + dr) + dn + 2 * i;
        TA* o = qw + (size_t)h * qo_hstride + 2 * i;
        const int n = min(2, dr - 2 * i);
        if (!ZLM_CHK(p, n * sizeof(TA)) || !ZLM_CHK(o, n * sizeof(TA))) continue;
        if (i < ang) {
            const float u = to_f32(p[0]), v = to_f32(p[1]);
            o[0] = from_f32<TA>(u * cs[0][i] - v * cs[1][i]);
            o[1] = from_f32<TA>(v * cs[0][i] + u * cs[1][i]);
        } else if (o != p) {
            o[0] = p[0];
            if (n > 1) o[1] = p[1];
        }
    }
    if (dkv == nullptr) return;
    if (!ZLM_CHK(token_slot + t, 4)) return;
    const int slot = token_slot[t];
    if (!ZLM_CHK(block_table + (size_t)slot * table_stride + pos / ZLM_PAGE, 4)) return;
    const int page = block_table[(size_t)slot * table_stride + pos / ZLM_PAGE];
    const TA* src = dkv + (size_t)t * dkv_stride;
    TA* rec = pool + ((size_t)page * ZLM_PAGE + pos % ZLM_PAGE) * (r + dr);
    if (!ZLM_CHK(src, (size_t)(r + dr) * sizeof(TA)) || !ZLM_CHK(rec, (size_t)(r + dr) * sizeof(TA))) return;
    TA* row = rec_out ? rec_out + (size_t)t * rec_stride : nullptr;
    if (row && !ZLM_CHK(row, (size_t)(r + dr) * sizeof(TA))) return;
    float ss = 0.f;
    for (int i = threadIdx.x; i < r; i += blockDim.x) {
        const float a = to_f32(src[i]);
        ss = fmaf(a, a, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)r + eps);
    for (int i = threadIdx.x; i < r; i += blockDim.x) {
        const TA c = from_f32<TA>((to_f32(src[i]) * inv) * cw[i]);
        rec[i] = c;
        if (row) row[i] = c;
    }
    for (int i = threadIdx.x; i < ang; i += blockDim.x) {
        const float u = to_f32(src[r + 2 * i]), v = to_f32(src[r + 2 * i + 1]);
        const TA a = from_f32<TA>(u * cs[0][i] - v * cs[1][i]), b = from_f32<TA>(v * cs[0][i] + u * cs[1][i]);
        rec[r + 2 * i] = a;
        rec[r + 2 * i + 1] = b;
        if (row) { row[r + 2 * i] = a; row[r + 2 * i + 1] = b; }
    }
    for (int i = n_rot + threadIdx.x; i < dr; i += blockDim.x) {
        rec[r + i] = src[r + i];
        if (row) row[r + i] = src[r + i];
    }
}

extern "C" int zlm_latent_prep(const void* q, int q_stride, void* qo, int qo_stride, int qo_hstride, const void* dkv,
                               int dkv_stride, int dtype, const void* cw,
                               int cw_dtype, float eps, const float* inv_freq, int n_rot, const int* token_pos,
                               const int* token_slot, const int* block_table, int table_stride, void* pool, int T,
                               int H, int dn, int dr, int r, void* rec_out, int rec_stride, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(rec_out == nullptr || (dkv != nullptr && rec_stride >= r + dr), "latent_prep: the records' second place needs "
                "the projection and rows of at least %d elements", r + dr);
    ZLM_REQUIRE(H > 0 && dn >= 0 && dr >= 0 && r > 0, "latent_prep: bad sizes heads=%d dim=%d rot_dim=%d kv_rank=%d", H, dn, dr, r);
    ZLM_REQUIRE(n_rot >= 0 && n_rot % 2 == 0 && n_rot <= dr && n_rot <= 512,
                "latent_prep: %d rotated dimensions of %d (even, at most 512)", n_rot, dr);
    ZLM_REQUIRE(n_rot == 0 || inv_freq, "latent_prep: the frequency table is missing");
    ZLM_REQUIRE(dkv == nullptr || (pool && block_table && token_slot && cw), "latent_prep: nowhere to write the records");
    VecW w{cw, cw_dtype};
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(latent_prep_kernel<float>, T, 128, 0, st, (const float*)q, q_stride, (float*)qo, qo_stride, qo_hstride,
                   (const float*)dkv, dkv_stride, w, eps,
                   inv_freq, n_rot, token_pos, token_slot, block_table, table_stride, (float*)pool, H, dn, dr, r,
                   (float*)rec_out, rec_stride);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(latent_prep_kernel<__nv_bfloat16>, T, 128, 0, st, (const __nv_bfloat16*)q, q_stride,
                   (__nv_bfloat16*)qo, qo_stride, qo_hstride, (const __nv_bfloat16*)dkv, dkv_stride, w, eps, inv_freq, n_rot, token_pos, token_slot, block_table,
                   table_stride, (__nv_bfloat16*)pool, H, dn, dr, r, (__nv_bfloat16*)rec_out, rec_stride);
    else
        ZLM_REQUIRE(false, "latent_prep: unsupported dtype %d", dtype);
    return zlm_check_launch("latent_prep");
}

// ---------------------------------------------------------------------------- per-head products
// out[t, h, n] = sum_k x[t, h, k] * W[h, n, k]; a warp owns one (h, n) and eight tokens at a time, its lanes
// share k, so a sum's order depends on K (and the operands' alignment) alone, never on the batch.
#define HL_TOK 8
__device__ __forceinline__ void hl_load4(const float* p, float* f) {
    const float4 v = *(const float4*)p;
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void hl_load4(const __nv_bfloat16* p, float* f) {
    const uint2 v = *(const uint2*)p;
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
}

// VEC: K and the strides are multiples of 4 and the operands aligned for loads of four elements: a lane takes
// four neighbouring k at a time (one load of W for eight tokens' loads of x); else one k at a time.
template <typename TA, bool VEC>
__global__ void __launch_bounds__(128)
head_linear_kernel(TA* __restrict__ out, int out_stride, int out_hstride, const TA* __restrict__ x, int x_stride,
                   int x_hstride, const TA* __restrict__ W, int T, int H, int N, int K) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * 4 + warp, h = blockIdx.y;
    if (n >= N) return;
    const TA* w = W + ((size_t)h * N + n) * K;
    pdl_wait();
    for (int t0 = blockIdx.z * HL_TOK; t0 < T; t0 += gridDim.z * HL_TOK) {
        float acc[HL_TOK];
#pragma unroll
        for (int j = 0; j < HL_TOK; ++j) acc[j] = 0.f;
        if (VEC) {
            for (int k = lane * 4; k < K; k += 128) {
                if (!ZLM_CHK(w + k, 4 * sizeof(TA))) continue;
                float wv[4], xv[4];
                hl_load4(w + k, wv);
#pragma unroll
                for (int j = 0; j < HL_TOK; ++j) {
                    const int t = t0 + j;
                    const TA* xp = x + (size_t)t * x_stride + (size_t)h * x_hstride + k;
                    if (t < T && ZLM_CHK(xp, 4 * sizeof(TA))) {
                        hl_load4(xp, xv);
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[j] = fmaf(xv[i], wv[i], acc[j]);
                    }
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) {
                if (!ZLM_CHK(w + k, sizeof(TA))) continue;
                const float wv = to_f32(w[k]);
#pragma unroll
                for (int j = 0; j < HL_TOK; ++j) {
                    const int t = t0 + j;
                    if (t < T && ZLM_CHK(x + (size_t)t * x_stride + (size_t)h * x_hstride + k, sizeof(TA)))
                        acc[j] = fmaf(to_f32(x[(size_t)t * x_stride + (size_t)h * x_hstride + k]), wv, acc[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < HL_TOK; ++j) {
            const float s = warp_sum(acc[j]);
            const int t = t0 + j;
            if (lane == 0 && t < T && ZLM_CHK(out + (size_t)t * out_stride + (size_t)h * out_hstride + n, sizeof(TA)))
                out[(size_t)t * out_stride + (size_t)h * out_hstride + n] = from_f32<TA>(s);
        }
    }
}

template <typename TA>
static void launch_head_linear(dim3 grid, cudaStream_t st, void* out, int out_stride, int out_hstride, const void* x,
                               int x_stride, int x_hstride, const void* W, int T, int H, int N, int K) {
    const size_t quad = 4 * sizeof(TA);
    const bool vec = K % 4 == 0 && x_stride % 4 == 0 && x_hstride % 4 == 0 && (uintptr_t)x % quad == 0 && (uintptr_t)W % quad == 0;
    if (vec)
        zlm_launch(head_linear_kernel<TA, true>, grid, 128, 0, st, (TA*)out, out_stride, out_hstride, (const TA*)x, x_stride,
                   x_hstride, (const TA*)W, T, H, N, K);
    else
        zlm_launch(head_linear_kernel<TA, false>, grid, 128, 0, st, (TA*)out, out_stride, out_hstride, (const TA*)x, x_stride,
                   x_hstride, (const TA*)W, T, H, N, K);
}

extern "C" int zlm_head_linear(void* out, int out_stride, int out_hstride, const void* x, int x_stride, int x_hstride,
                               const void* W, int dtype, int T, int H, int N, int K, cudaStream_t st) {
    if (T == 0 || N == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && H > 0 && H <= 65535 && N > 0 && K > 0, "head_linear: bad sizes T=%d heads=%d N=%d K=%d", T, H, N, K);
    int tz = (T + HL_TOK - 1) / HL_TOK;
    if (tz > 64) tz = 64;
    dim3 grid((N + 3) / 4, H, tz);
    if (dtype == ZLM_DTYPE_F32)
        launch_head_linear<float>(grid, st, out, out_stride, out_hstride, x, x_stride, x_hstride, W, T, H, N, K);
    else if (dtype == ZLM_DTYPE_BF16)
        launch_head_linear<__nv_bfloat16>(grid, st, out, out_stride, out_hstride, x, x_stride, x_hstride, W, T, H, N, K);
    else
        ZLM_REQUIRE(false, "head_linear: unsupported dtype %d", dtype);
    return zlm_check_launch("head_linear");
}

// ---------------------------------------------------------------------------- attention, any size
// One block per (token, head).  The keys are walked in chunks of 32 aligned to absolute positions
// and dealt round-robin to the 4 warps (a lane takes one key of the chunk), then the warps are merged
// in a fixed order.  q is [T, H, r + dr] (folded query | rotated part), out [T, H, r].  `sinks` (optional): one
// number per head whose exponential joins the softmax's denominator without a value; `chunk`: only the keys of the
// query's own chunk of that many positions, counted from position 0.
#define LAT_WARPS 4
template <typename TA, int NPL>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_attention_kernel(TA* __restrict__ out, int out_stride, const TA* __restrict__ q, int q_stride,
                        const TA* __restrict__ pool, const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ token_pos, const int* __restrict__ token_slot, int H, int r, int dr,
                        float scale, int window, int chunk, const float* __restrict__ sinks) {
    extern __shared__ float sm[];
    const int D = r + dr;
    float* qs = sm;                         // [D]
    float* accs = sm + D;                   // [LAT_WARPS][r]
    __shared__ float ms[LAT_WARPS], ls[LAT_WARPS];
    pdl_launch_dependents();
    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(token_slot + t, 4)) return;
    const int pos = token_pos[t], slot = token_slot[t];
    const int seq = pos + 1;
    int t_start = (window != 0 && seq > window) ? seq - window : 0;
    if (chunk > 0) t_start = max(t_start, pos - pos % chunk);
    const int* pages = block_table + (size_t)slot * table_stride;
    pdl_wait();
    const TA* qp = q + (size_t)t * q_stride + (size_t)h * D;
    TA* op = out + (size_t)t * out_stride + (size_t)h * r;
    if (!ZLM_CHK(qp, (size_t)D * sizeof(TA)) || !ZLM_CHK(op, (size_t)r * sizeof(TA))) return;
    for (int e = threadIdx.x; e < D; e += blockDim.x) qs[e] = to_f32(qp[e]);
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    if (sinks && warp == 0 && ZLM_CHK(sinks + h, 4)) { m = sinks[h]; l = 1.f; }      // exp(sinks[h]): a term without a value
    float acc[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) acc[i] = 0.f;
    const int c0 = t_start / 32, c1 = pos / 32;
    for (int c = c0 + ((warp - c0 % LAT_WARPS + LAT_WARPS) % LAT_WARPS); c <= c1; c += LAT_WARPS) {
        const int key = c * 32 + lane;
        const bool valid = key >= t_start && key <= pos;
        if (!ZLM_CHK(pages + (c * 32) / ZLM_PAGE, 4)) continue;
        const int page = pages[(c * 32) / ZLM_PAGE];
        const TA* base = pool + (size_t)page * ZLM_PAGE * D;
        if (!ZLM_CHK(base, (size_t)ZLM_PAGE * D * sizeof(TA))) continue;
        float s = -INFINITY;
        if (valid) {
            const TA* kr = base + (size_t)(key % ZLM_PAGE) * D;
            float d = 0.f;
            for (int e = 0; e < D; ++e) d = fmaf(qs[e], to_f32(kr[e]), d);
            s = d * scale;
        }
        const float cm = warp_max(s);
        const float mn = fmaxf(m, cm);
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - mn);
        const float p = valid ? expf(s - mn) : 0.f;
        l = l * alpha + warp_sum(p);
        m = mn;
#pragma unroll
        for (int i = 0; i < NPL; ++i) acc[i] *= alpha;
        const int hi = min(31, pos - c * 32), lo = max(0, t_start - c * 32);
        for (int jk = lo; jk <= hi; ++jk) {
            const float pj = __shfl_sync(0xffffffffu, p, jk);
            const TA* vr = base + (size_t)((c * 32 + jk) % ZLM_PAGE) * D;
#pragma unroll
            for (int i = 0; i < NPL; ++i) {
                const int e = lane + 32 * i;
                if (e < r) acc[i] = fmaf(pj, to_f32(vr[e]), acc[i]);
            }
        }
    }
    if (lane == 0) { ms[warp] = m; ls[warp] = l; }
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int e = lane + 32 * i;
        if (e < r) accs[warp * r + e] = acc[i];
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < LAT_WARPS; ++w) M = fmaxf(M, ms[w]);
    float L = 0.f, f[LAT_WARPS];
#pragma unroll
    for (int w = 0; w < LAT_WARPS; ++w) {
        f[w] = (ms[w] == -INFINITY) ? 0.f : expf(ms[w] - M);
        L += ls[w] * f[w];
    }
    const float invL = 1.0f / L;
    for (int e = threadIdx.x; e < r; e += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < LAT_WARPS; ++w) o += accs[w * r + e] * f[w];
        op[e] = from_f32<TA>(o * invL);
    }
}

template <typename TA>
static int launch_latent_attention(void* out, int out_stride, const void* q, int q_stride, const void* pool,
                                   const int* block_table, int table_stride, const int* token_pos, const int* token_slot,
                                   int T, int H, int r, int dr, float scale, int window, int chunk, const float* sinks,
                                   cudaStream_t st) {
    dim3 grid(T, H);
    const size_t smem = (size_t)(r + dr + LAT_WARPS * r) * sizeof(float);
#define ZLM_LAT(NPL)                                                                                                  \
    do {                                                                                                              \
        static bool big[64] = {};                                                                                     \
        if (smem > 48 * 1024 && !big[zlm_device_index()]) {                                                           \
            cudaFuncSetAttribute(latent_attention_kernel<TA, NPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
            big[zlm_device_index()] = true;                                                                           \
        }                                                                                                             \
        zlm_launch(latent_attention_kernel<TA, NPL>, grid, LAT_WARPS * 32, smem, st, (TA*)out, out_stride, (const TA*)q, \
                   q_stride, (const TA*)pool, block_table, table_stride, token_pos, token_slot, H, r, dr, scale, window, chunk, sinks); \
    } while (0)
    if (r <= 128) ZLM_LAT(4);
    else if (r <= 512) ZLM_LAT(16);
    else ZLM_LAT(32);
#undef ZLM_LAT
    return zlm_check_launch("latent_attention");
}

extern "C" int zlm_latent_attention(void* out, int out_stride, const void* q, int q_stride, int dtype, const void* pool,
                                    const int* block_table, int table_stride, const int* token_pos,
                                    const int* token_slot, int T, int H, int r, int dr, float scale, int window,
                                    int chunk, const float* sinks, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(H > 0 && H <= 65535 && r > 0 && r <= 1024 && dr >= 0 && dr <= 1024,
                "latent_attention: heads=%d kv_rank=%d rot_dim=%d (kv_rank and rot_dim at most 1024)", H, r, dr);
    ZLM_REQUIRE(window >= 0 && chunk >= 0, "latent_attention: window=%d chunk=%d", window, chunk);
    if (dtype == ZLM_DTYPE_F32)
        return launch_latent_attention<float>(out, out_stride, q, q_stride, pool, block_table, table_stride, token_pos,
                                              token_slot, T, H, r, dr, scale, window, chunk, sinks, st);
    if (dtype == ZLM_DTYPE_BF16)
        return launch_latent_attention<__nv_bfloat16>(out, out_stride, q, q_stride, pool, block_table, table_stride,
                                                      token_pos, token_slot, T, H, r, dr, scale, window, chunk, sinks, st);
    ZLM_REQUIRE(false, "latent_attention: unsupported dtype %d", dtype);
    return ZLM_OK;
}

// ---------------------------------------------------------------------------- unfolded keys and values of a step
// For whole prompts the per-head keys and values of the step's own tokens may be written out once, so that the
// library's flash attention over per-head keys and values serves the step (fewer flops than the folded form by
// (kv_rank + rot_dim + kv_rank) / (dim + rot_dim + v_dim)):
//   latent_gather    rec[t, :] = the record of token t from the paged pool
//   latent_unfold    K[page, h, place, :] = [kn[t, h, :dn] | kr[t, :dr]],  V[page, h, place, :] = [v[t, h, :dv] | 0]
//                    into a pool of the attention kernels' layout [pages, 2, H, 64, hd], hd = dn + dr, pages by a
//                    table of the step's own (row = the sequence's number in the step)
template <typename TA>
__global__ void __launch_bounds__(128)
latent_gather_kernel(TA* __restrict__ rec, const TA* __restrict__ pool, const int* __restrict__ block_table,
                     int table_stride, const int* __restrict__ token_pos, const int* __restrict__ token_slot, int R) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(token_slot + t, 4)) return;
    const int pos = token_pos[t], slot = token_slot[t];
    if (!ZLM_CHK(block_table + (size_t)slot * table_stride + pos / ZLM_PAGE, 4)) return;
    const int page = block_table[(size_t)slot * table_stride + pos / ZLM_PAGE];
    pdl_wait();
    const TA* src = pool + ((size_t)page * ZLM_PAGE + pos % ZLM_PAGE) * R;
    TA* dst = rec + (size_t)t * R;
    for (int i = threadIdx.x; i < R; i += blockDim.x)
        if (ZLM_CHK(src + i, sizeof(TA)) && ZLM_CHK(dst + i, sizeof(TA))) dst[i] = src[i];
}

template <typename TA>
__global__ void __launch_bounds__(256)
latent_unfold_kernel(TA* __restrict__ spool, const int* __restrict__ stable, int stable_stride, const TA* __restrict__ kv,
                     int kv_stride, const TA* __restrict__ rec, int rec_stride, const int* __restrict__ token_pos,
                     const int* __restrict__ token_seq, int H, int dn, int dr, int dv, int r) {
    pdl_launch_dependents();
    const int t = blockIdx.x, hd = dn + dr;
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(token_seq + t, 4)) return;
    const int pos = token_pos[t], seq = token_seq[t];
    if (!ZLM_CHK(stable + (size_t)seq * stable_stride + pos / ZLM_PAGE, 4)) return;
    const int page = stable[(size_t)seq * stable_stride + pos / ZLM_PAGE];
    pdl_wait();
    const size_t tile = (size_t)ZLM_PAGE * hd;
    TA* kbase = spool + (size_t)page * 2 * H * tile + (size_t)(pos % ZLM_PAGE) * hd;
    TA* vbase = kbase + (size_t)H * tile;
    const TA* kvr = kv + (size_t)t * kv_stride;
    const TA* kr = rec + (size_t)t * rec_stride + r;
    for (int e = threadIdx.x; e < H * hd; e += blockDim.x) {
        const int h = e / hd, i = e - h * hd;
        TA* kd = kbase + (size_t)h * tile + i;
        TA* vd = vbase + (size_t)h * tile + i;
        if (!ZLM_CHK(kd, sizeof(TA)) || !ZLM_CHK(vd, sizeof(TA))) continue;
        const TA* ks = i < dn ? kvr + (size_t)h * dn + i : kr + (i - dn);
        *kd = ZLM_CHK(ks, sizeof(TA)) ? *ks : from_f32<TA>(0.f);
        const TA* vs = kvr + (size_t)H * dn + (size_t)h * dv + i;
        *vd = (i < dv && ZLM_CHK(vs, sizeof(TA))) ? *vs : from_f32<TA>(0.f);
    }
}

// the same in pieces of 8 elements (16 bytes), for bfloat16 with every width a multiple of 8: a thread copies a piece
// of a head's key and the piece of its value at the same columns
__global__ void __launch_bounds__(256)
latent_unfold_v8_kernel(__nv_bfloat16* __restrict__ spool, const int* __restrict__ stable, int stable_stride,
                        const __nv_bfloat16* __restrict__ kv, int kv_stride, const __nv_bfloat16* __restrict__ rec,
                        int rec_stride, const int* __restrict__ token_pos, const int* __restrict__ token_seq, int H, int dn,
                        int dr, int dv, int r) {
    pdl_launch_dependents();
    const int t = blockIdx.x, hd = dn + dr, per = hd / 8;
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(token_seq + t, 4)) return;
    const int pos = token_pos[t], seq = token_seq[t];
    if (!ZLM_CHK(stable + (size_t)seq * stable_stride + pos / ZLM_PAGE, 4)) return;
    const int page = stable[(size_t)seq * stable_stride + pos / ZLM_PAGE];
    pdl_wait();
    const size_t tile = (size_t)ZLM_PAGE * hd;
    __nv_bfloat16* kbase = spool + (size_t)page * 2 * H * tile + (size_t)(pos % ZLM_PAGE) * hd;
    __nv_bfloat16* vbase = kbase + (size_t)H * tile;
    const __nv_bfloat16* kvr = kv + (size_t)t * kv_stride;
    const __nv_bfloat16* kr = rec + (size_t)t * rec_stride + r;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int c = threadIdx.x; c < H * per; c += blockDim.x) {
        const int h = c / per, i = (c - h * per) * 8;
        __nv_bfloat16* kd = kbase + (size_t)h * tile + i;
        __nv_bfloat16* vd = vbase + (size_t)h * tile + i;
        if (!ZLM_CHK(kd, 16) || !ZLM_CHK(vd, 16)) continue;
        const __nv_bfloat16* ks = i < dn ? kvr + (size_t)h * dn + i : kr + (i - dn);
        *(uint4*)kd = ZLM_CHK(ks, 16) ? *(const uint4*)ks : zero;
        const __nv_bfloat16* vs = kvr + (size_t)H * dn + (size_t)h * dv + i;
        *(uint4*)vd = (i < dv && ZLM_CHK(vs, 16)) ? *(const uint4*)vs : zero;
    }
}

extern "C" int zlm_latent_gather(void* rec, const void* pool, const int* block_table, int table_stride,
                                 const int* token_pos, const int* token_slot, int dtype, int T, int R, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0, "latent_gather: record of %d elements", R);
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(latent_gather_kernel<float>, T, 128, 0, st, (float*)rec, (const float*)pool, block_table, table_stride,
                   token_pos, token_slot, R);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(latent_gather_kernel<__nv_bfloat16>, T, 128, 0, st, (__nv_bfloat16*)rec, (const __nv_bfloat16*)pool,
                   block_table, table_stride, token_pos, token_slot, R);
    else
        ZLM_REQUIRE(false, "latent_gather: unsupported dtype %d", dtype);
    return zlm_check_launch("latent_gather");
}

extern "C" int zlm_latent_unfold(void* spool, const int* stable, int stable_stride, const void* kv, int kv_stride,
                                 const void* rec, int rec_stride, const int* token_pos, const int* token_seq, int dtype,
                                 int T, int H, int dn, int dr, int dv, int r, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(H > 0 && dn >= 0 && dr >= 0 && dn + dr > 0 && dv > 0 && dv <= dn + dr && r > 0,
                "latent_unfold: heads=%d dim=%d rot_dim=%d v_dim=%d", H, dn, dr, dv);
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(latent_unfold_kernel<float>, T, 256, 0, st, (float*)spool, stable, stable_stride, (const float*)kv, kv_stride,
                   (const float*)rec, rec_stride, token_pos, token_seq, H, dn, dr, dv, r);
    else if (dtype == ZLM_DTYPE_BF16 && dn % 8 == 0 && dr % 8 == 0 && dv % 8 == 0 && r % 8 == 0 && kv_stride % 8 == 0 &&
             rec_stride % 8 == 0 && (uintptr_t)spool % 16 == 0 && (uintptr_t)kv % 16 == 0 && (uintptr_t)rec % 16 == 0)
        zlm_launch(latent_unfold_v8_kernel, T, 256, 0, st, (__nv_bfloat16*)spool, stable, stable_stride,
                   (const __nv_bfloat16*)kv, kv_stride, (const __nv_bfloat16*)rec, rec_stride, token_pos, token_seq, H, dn, dr,
                   dv, r);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(latent_unfold_kernel<__nv_bfloat16>, T, 256, 0, st, (__nv_bfloat16*)spool, stable, stable_stride,
                   (const __nv_bfloat16*)kv, kv_stride, (const __nv_bfloat16*)rec, rec_stride, token_pos, token_seq, H, dn, dr,
                   dv, r);
    else
        ZLM_REQUIRE(false, "latent_unfold: unsupported dtype %d", dtype);
    return zlm_check_launch("latent_unfold");
}

ZLM_TRANSLATION_UNIT(latent_attention)
