// Differential attention around the library's attention kernels: every head has two attention maps over the same
// values, o = a1 - lambda * a2, followed by a unit norm per head.
//
// The two maps run as two query heads and two key heads of the ordinary grouped attention that share one value head
// (the kernels' `v_share` = 2).  With H query heads over G key/value heads (rep = H / G) the attention sees
//   query head  (g * 2 + m) * rep + j   = map m of head g * rep + j
//   key head     g * 2 + m              = map m of key head g
//   value head   g                      (page layout [2G key heads | G value heads] of [ZLM_PAGE][hdp])
// so that query head i reads key head i / rep as always.  Keys (width dim) and values (width vdim) are padded with
// zeros to one width hdp.
//
//   diff_prep     on the fused projection [q: H*2*dim | k: G*2*dim | v: G*vdim] of every token: RMS norm of every
//                 map of q and k over dim (one weight for q, one for k), rotation of neighbouring pairs (2i, 2i+1),
//                 i < n_rot/2, by pos * inv_freq[i]; q to q_out [T, 2H, hdp] in the order above, k and v to the
//                 token's place in the paged pool.  Norm, angle, sine and cosine in fp32.
//   diff_combine  out[t, h, :vdim] = unit_rms(a1 - lambda * a2) * post, from the attention's output [T, 2H, hdp]
#include "common.cuh"

#define DIFF_WARPS 4

template <typename TA>
__global__ void __launch_bounds__(DIFF_WARPS * 32)
diff_prep_kernel(TA* __restrict__ q_out, int q_out_stride, const TA* __restrict__ proj, int proj_stride, VecW q_w, VecW k_w,
                 float eps, const float* __restrict__ inv_freq, int n_rot, const int* __restrict__ token_pos,
                 const int* __restrict__ token_slot, const int* __restrict__ block_table, int table_stride,
                 TA* __restrict__ pool, int T, int H, int G, int dim, int vdim, int hdp) {
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int units = 2 * H + 3 * G;                 // q maps, k maps, v heads of one token
    const int t = blockIdx.x;
    const int u = blockIdx.y * DIFF_WARPS + warp;
    if (u >= units) return;
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(token_slot + t, 4)) return;
    const int pos = token_pos[t], slot = token_slot[t];
    const int rep = H / G;
    const TA* row = proj + (size_t)t * proj_stride;
    // where the unit's numbers come from, how wide they are, and where they go
    const TA* src;
    TA* dst;
    int width;
    bool normed;
    VecW w = q_w;
    const size_t place = (size_t)(pos % ZLM_PAGE) * hdp;
    size_t page_base = 0;
    if (u >= 2 * H) {
        if (!ZLM_CHK(block_table + (size_t)slot * table_stride + pos / ZLM_PAGE, 4)) return;
        page_base = (size_t)block_table[(size_t)slot * table_stride + pos / ZLM_PAGE] * (size_t)(3 * G) * ZLM_PAGE * hdp;
    }
    if (u < 2 * H) {
        const int h = u >> 1, m = u & 1;             // the projection's order: head by head [map 0 | map 1]
        const int g = h / rep, j = h % rep;
        src = row + (size_t)u * dim;
        dst = q_out + (size_t)t * q_out_stride + (size_t)((g * 2 + m) * rep + j) * hdp;
        width = dim;
        normed = true;
    } else if (u < 2 * H + 2 * G) {
        const int kh = u - 2 * H;                    // g * 2 + m
        src = row + (size_t)2 * H * dim + (size_t)kh * dim;
        dst = pool + page_base + (size_t)kh * ZLM_PAGE * hdp + place;
        width = dim;
        normed = true;
        w = k_w;
    } else {
        const int g = u - 2 * H - 2 * G;
        src = row + (size_t)(2 * H + 2 * G) * dim + (size_t)g * vdim;
        dst = pool + page_base + (size_t)(2 * G + g) * ZLM_PAGE * hdp + place;
        width = vdim;
        normed = false;
    }
    pdl_wait();
    if (!ZLM_CHK(src, (size_t)width * sizeof(TA)) || !ZLM_CHK(dst, (size_t)hdp * sizeof(TA))) return;
    if (!normed) {
        for (int e = lane; e < hdp; e += 32) dst[e] = e < width ? src[e] : from_f32<TA>(0.f);
        return;
    }
    float ss = 0.f;
    for (int e = lane; e < width; e += 32) {
        const float a = to_f32(src[e]);
        ss = fmaf(a, a, ss);
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)width + eps);
    // a lane owns pairs (2p, 2p + 1): the rotation's partners
    for (int p = lane; 2 * p < hdp; p += 32) {
        const int e0 = 2 * p, e1 = 2 * p + 1;
        float a = e0 < width ? (to_f32(src[e0]) * inv) * w[e0] : 0.f;
        float b = e1 < width ? (to_f32(src[e1]) * inv) * w[e1] : 0.f;
        if (e1 < n_rot) {
            float sn, cs;
            sincosf((float)pos * inv_freq[p], &sn, &cs);
            const float ra = a * cs - b * sn, rb = b * cs + a * sn;
            a = ra;
            b = rb;
        }
        dst[e0] = from_f32<TA>(a);
        if (e1 < hdp) dst[e1] = from_f32<TA>(b);
    }
}

extern "C" int zlm_diff_prep(void* q_out, int q_out_stride, const void* proj, int proj_stride, int dtype, const void* q_w,
                             const void* k_w, int w_dtype, float eps, const float* inv_freq, int n_rot,
                             const int* token_pos, const int* token_slot, const int* block_table, int table_stride,
                             void* pool, int T, int H, int G, int dim, int vdim, int hdp, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && hdp >= dim && hdp >= vdim && hdp % 2 == 0,
                "diff_prep: %d heads over %d, dim=%d vdim=%d padded to %d", H, G, dim, vdim, hdp);
    ZLM_REQUIRE(n_rot >= 0 && n_rot % 2 == 0 && n_rot <= dim && (n_rot == 0 || inv_freq), "diff_prep: n_rot=%d of %d", n_rot, dim);
    const int units = 2 * H + 3 * G;
    ZLM_REQUIRE((units + DIFF_WARPS - 1) / DIFF_WARPS <= 65535, "diff_prep: too many heads");
    const dim3 grid(T, (units + DIFF_WARPS - 1) / DIFF_WARPS), block(DIFF_WARPS * 32);
    VecW qw{q_w, w_dtype}, kw{k_w, w_dtype};
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(diff_prep_kernel<float>, grid, block, 0, st, (float*)q_out, q_out_stride, (const float*)proj, proj_stride, qw,
                   kw, eps, inv_freq, n_rot, token_pos, token_slot, block_table, table_stride, (float*)pool, T, H, G, dim,
                   vdim, hdp);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(diff_prep_kernel<__nv_bfloat16>, grid, block, 0, st, (__nv_bfloat16*)q_out, q_out_stride,
                   (const __nv_bfloat16*)proj, proj_stride, qw, kw, eps, inv_freq, n_rot, token_pos, token_slot, block_table,
                   table_stride, (__nv_bfloat16*)pool, T, H, G, dim, vdim, hdp);
    else
        ZLM_REQUIRE(false, "diff_prep: unsupported dtype %d", dtype);
    return zlm_check_launch("diff_prep");
}

// a warp per (token, head): a1 and a2 are the attention's outputs of the head's two maps
template <typename TA>
__global__ void __launch_bounds__(DIFF_WARPS * 32)
diff_combine_kernel(TA* __restrict__ out, int out_stride, const TA* __restrict__ a, int a_stride, int T, int H, int G,
                    int vdim, int hdp, float lambda, float post, float eps) {
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x, h = blockIdx.y * DIFF_WARPS + warp;
    if (h >= H) return;
    const int rep = H / G, g = h / rep, j = h % rep;
    const TA* a1 = a + (size_t)t * a_stride + (size_t)((g * 2) * rep + j) * hdp;
    const TA* a2 = a + (size_t)t * a_stride + (size_t)((g * 2 + 1) * rep + j) * hdp;
    TA* dst = out + (size_t)t * out_stride + (size_t)h * vdim;
    pdl_wait();
    if (!ZLM_CHK(a1, (size_t)vdim * sizeof(TA)) || !ZLM_CHK(a2, (size_t)vdim * sizeof(TA)) || !ZLM_CHK(dst, (size_t)vdim * sizeof(TA)))
        return;
    float ss = 0.f;
    for (int e = lane; e < vdim; e += 32) {
        const float d = to_f32(a1[e]) - lambda * to_f32(a2[e]);
        ss = fmaf(d, d, ss);
    }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    for (int e = lane; e < vdim; e += 32) {
        const float d = to_f32(a1[e]) - lambda * to_f32(a2[e]);
        dst[e] = from_f32<TA>((d * inv) * post);
    }
}

extern "C" int zlm_diff_combine(void* out, int out_stride, const void* a, int a_stride, int dtype, int T, int H, int G,
                                int vdim, int hdp, float lambda, float post, float eps, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(H > 0 && G > 0 && H % G == 0 && vdim > 0 && hdp >= vdim && (H + DIFF_WARPS - 1) / DIFF_WARPS <= 65535,
                "diff_combine: %d heads over %d, vdim=%d padded to %d", H, G, vdim, hdp);
    const dim3 grid(T, (H + DIFF_WARPS - 1) / DIFF_WARPS), block(DIFF_WARPS * 32);
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(diff_combine_kernel<float>, grid, block, 0, st, (float*)out, out_stride, (const float*)a, a_stride, T, H, G,
                   vdim, hdp, lambda, post, eps);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(diff_combine_kernel<__nv_bfloat16>, grid, block, 0, st, (__nv_bfloat16*)out, out_stride,
                   (const __nv_bfloat16*)a, a_stride, T, H, G, vdim, hdp, lambda, post, eps);
    else
        ZLM_REQUIRE(false, "diff_combine: unsupported dtype %d", dtype);
    return zlm_check_launch("diff_combine");
}

ZLM_TRANSLATION_UNIT(diff_attention)
