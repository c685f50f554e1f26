// Operations on the fp32 residual stream and around it that designs with a norm on the sublayer's *output* need:
//   embed_scaled     out[t] = table[id_t] * scale (+ pair[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets], a second
//                    table looked up by the token and the token before it; the row `buckets` for a sequence's first
//                    token).  The token before a step's first one is per-slot state.
//   norm_scale_add   stream[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w (* ls): RMS norm of a sublayer's output, an
//                    optional second vector (a scale per coordinate of the layer), and the residual add, all in fp32
//   cast_rows        the stream's rows rounded to the compute dtype (the input of a sublayer that reads the stream
//                    itself, without a norm before it)
//   gated_act        out[t, i] = act(gu[t, i]) * gu[t, I + i], act = silu or the tanh form of gelu
//   scale_f32        x *= s (logits times a constant)
//   head_scalar_gate x[t, h, :] *= sigmoid(g[t, h]): one gate number per head
#include "common.cuh"
#include "elementwise.cuh"

// ---------------------------------------------------------------- embedding with a scale and a pair table
template <typename TW>
__global__ void embed_scaled_kernel(float* __restrict__ out, const TW* __restrict__ table, float scale,
                                    const TW* __restrict__ pair, int buckets, long long mul_prev, long long mul_cur,
                                    const int* __restrict__ ids, const int* __restrict__ token_pos,
                                    const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                                    const int* __restrict__ seq_slot, int* __restrict__ prev_state, int H, int V) {
    __shared__ int s_row;
    pdl_trigger();
    const int t = blockIdx.x;
    pdl_wait();                 // the ids may be what the previous step's sampler wrote
    if (!ZLM_CHK(ids + t, 4) || !ZLM_CHK(out + (size_t)t * H, (size_t)H * 4)) return;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);       // ids are validated on the host; a bad one never reads outside
    if (pair != nullptr && threadIdx.x == 0) {
        int row = buckets;
        if (ZLM_CHK(token_pos + t, 4) && ZLM_CHK(token_seq + t, 4)) {
            const int seq = token_seq[t];
            if (ZLM_CHK(cu_seqlens + seq, 8) && ZLM_CHK(seq_slot + seq, 4)) {
                const int first = cu_seqlens[seq], last = cu_seqlens[seq + 1] - 1;
                const int slot = seq_slot[seq];
                int prev = -1;
                if (t > first) {
                    prev = ZLM_CHK(ids + t - 1, 4) ? ids[t - 1] : -1;
                } else {
                    // the step's first token of this sequence: the token before it is the slot's state, which this
                    // same thread then replaces by the step's last token (nobody else reads or writes it)
                    if (token_pos[t] > 0 && ZLM_CHK(prev_state + slot, 4)) prev = prev_state[slot];
                    if (ZLM_CHK(prev_state + slot, 4) && ZLM_CHK(ids + last, 4)) prev_state[slot] = ids[last];
                }
                if (prev >= 0) row = (int)(((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets);
            }
        }
        s_row = row;
    }
    __syncthreads();
    const TW* er = table + (size_t)id * H;
    float* o = out + (size_t)t * H;
    if (!ZLM_CHK(er, (size_t)H * sizeof(TW))) return;
    if (pair != nullptr) {
        const TW* pr = pair + (size_t)s_row * H;
        if (!ZLM_CHK(pr, (size_t)H * sizeof(TW))) return;
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = fmaf(to_f32(er[i]), scale, to_f32(pr[i]));
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(er[i]) * scale;
    }
}

extern "C" int zlm_embed_scaled(float* out, const void* table, int dtype, float scale, const void* pair, int buckets,
                                long long mul_prev, long long mul_cur, const int* ids, const int* token_pos,
                                const int* token_seq, const int* cu_seqlens, const int* seq_slot, int* prev_state, int T,
                                int H, int V, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && H > 0 && V > 0, "embed_scaled: bad sizes T=%d H=%d V=%d", T, H, V);
    ZLM_REQUIRE(pair == nullptr || (buckets > 0 && mul_prev >= 0 && mul_cur >= 0 && token_pos && token_seq && cu_seqlens &&
                                    seq_slot && prev_state),
                "embed_scaled: the pair table needs buckets > 0, multipliers >= 0, the step's arrays and the slots' state");
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(embed_scaled_kernel<float>, T, threads, 0, st, out, (const float*)table, scale, (const float*)pair, buckets,
                   mul_prev, mul_cur, ids, token_pos, token_seq, cu_seqlens, seq_slot, prev_state, H, V);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(embed_scaled_kernel<__nv_bfloat16>, T, threads, 0, st, out, (const __nv_bfloat16*)table, scale,
                   (const __nv_bfloat16*)pair, buckets, mul_prev, mul_cur, ids, token_pos, token_seq, cu_seqlens, seq_slot,
                   prev_state, H, V);
    else
        ZLM_REQUIRE(false, "embed_scaled: unsupported table dtype %d", dtype);
    return zlm_check_launch("embed_scaled");
}

// ---------------------------------------------------------------- norm of a sublayer's output, scale, residual add
// One block per row; the block's size is a function of H alone, so the order of the sum of squares never depends on
// the batch.  With H a multiple of 4 and up to 4 float4 a thread the row is read once.  `cast_out` (may be null)
// receives the stream's new row rounded to bfloat16: what the next sublayer's products read.
template <typename TY>
__global__ void norm_scale_add_kernel(float* __restrict__ stream, const TY* __restrict__ y, VecW w, VecW ls, int has_ls,
                                      int H, float eps, __nv_bfloat16* __restrict__ cast_out) {
    __shared__ float red[32];
    pdl_trigger();
    const int r = blockIdx.x;
    pdl_wait();
    float* xr = stream + (size_t)r * H;
    const TY* yr = y + (size_t)r * H;
    if (!ZLM_CHK(xr, (size_t)H * 4) || !ZLM_CHK(yr, (size_t)H * sizeof(TY)) ||
        !ZLM_CHK(w.p, (size_t)H * (w.dtype == ZLM_DTYPE_F32 ? 4 : 2)) ||
        (has_ls && !ZLM_CHK(ls.p, (size_t)H * (ls.dtype == ZLM_DTYPE_F32 ? 4 : 2))) ||
        (cast_out && !ZLM_CHK(cast_out + (size_t)r * H, (size_t)H * 2)))
        return;
    __nv_bfloat16* cr = cast_out ? cast_out + (size_t)r * H : nullptr;
    const int nv = H / 4;
    const bool in_regs = sizeof(TY) == 4 && H % 4 == 0 && nv <= NORM_MAX_V4 * (int)blockDim.x;
    float4 v[NORM_MAX_V4];
    float s = 0.f;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < NORM_MAX_V4; ++j) {
            const int c = threadIdx.x + j * blockDim.x;
            v[j] = c < nv ? *(const float4*)((const float*)yr + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            s = fmaf(v[j].x, v[j].x, s); s = fmaf(v[j].y, v[j].y, s);
            s = fmaf(v[j].z, v[j].z, s); s = fmaf(v[j].w, v[j].w, s);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float a = to_f32(yr[i]);
            s = fmaf(a, a, s);
        }
    }
    const float tot = block_sum(s, red);
    const float inv = 1.0f / sqrtf(tot / (float)H + eps);
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < NORM_MAX_V4; ++j) {
            const int c = threadIdx.x + j * blockDim.x;
            if (c >= nv) continue;
            const int i = c * 4;
            float4 wv = w.load4(i);
            if (has_ls) {
                const float4 l = ls.load4(i);
                // (y * inv * w) * ls, in that order, as two roundings of the norm's result
                float4 a = *(float4*)(xr + i);
                a.x += ((v[j].x * inv) * wv.x) * l.x; a.y += ((v[j].y * inv) * wv.y) * l.y;
                a.z += ((v[j].z * inv) * wv.z) * l.z; a.w += ((v[j].w * inv) * wv.w) * l.w;
                *(float4*)(xr + i) = a;
                if (cr) store4(cr + i, a.x, a.y, a.z, a.w);
            } else {
                float4 a = *(float4*)(xr + i);
                a.x += (v[j].x * inv) * wv.x; a.y += (v[j].y * inv) * wv.y;
                a.z += (v[j].z * inv) * wv.z; a.w += (v[j].w * inv) * wv.w;
                *(float4*)(xr + i) = a;
                if (cr) store4(cr + i, a.x, a.y, a.z, a.w);
            }
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float n = (to_f32(yr[i]) * inv) * w[i];
            if (has_ls) n *= ls[i];
            const float a = xr[i] + n;
            xr[i] = a;
            if (cr) cr[i] = __float2bfloat16_rn(a);
        }
    }
}

extern "C" int zlm_norm_scale_add(float* stream, const void* y, int y_dtype, const void* w, int w_dtype, const void* ls,
                                  int ls_dtype, int R, int H, float eps, void* cast_out, cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0 && H > 0, "norm_scale_add: bad sizes R=%d H=%d", R, H);
    ZLM_REQUIRE(H % 4 != 0 || (uintptr_t)cast_out % 8 == 0, "norm_scale_add: the bfloat16 copy must be 8-byte aligned");
    ZLM_REQUIRE(H % 4 != 0 || ((uintptr_t)stream % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                               (uintptr_t)ls % 16 == 0),
                "norm_scale_add: stream, input and vectors must be 16-byte aligned");
    int threads = 128;
    while (threads < 1024 && threads * 4 * NORM_MAX_V4 < H) threads *= 2;
    VecW vw{w, w_dtype}, vl{ls ? ls : w, ls ? ls_dtype : w_dtype};
    if (y_dtype == ZLM_DTYPE_F32)
        zlm_launch(norm_scale_add_kernel<float>, R, threads, 0, st, stream, (const float*)y, vw, vl, ls ? 1 : 0, H, eps,
                   (__nv_bfloat16*)cast_out);
    else if (y_dtype == ZLM_DTYPE_BF16)
        zlm_launch(norm_scale_add_kernel<__nv_bfloat16>, R, threads, 0, st, stream, (const __nv_bfloat16*)y, vw, vl,
                   ls ? 1 : 0, H, eps, (__nv_bfloat16*)cast_out);
    else
        ZLM_REQUIRE(false, "norm_scale_add: unsupported input dtype %d", y_dtype);
    return zlm_check_launch("norm_scale_add");
}

// ---------------------------------------------------------------- the same, and the norm that reads the stream next
// stream += y / rms(y) * w1, then out2 = stream / rms(stream) * w2 in the element type: a layer that norms a sublayer's
// output and the next sublayer's input does both in one pass over the row, which is held in shared memory as fp32.
// One block per row, its size a function of H alone.
template <typename TO>
__global__ void norm_add_norm_kernel(float* __restrict__ stream, const float* __restrict__ y, VecW w1, float eps1,
                                     TO* __restrict__ out2, VecW w2, float eps2, int H, int in_regs) {
    extern __shared__ float nan_row[];          // [32] reduction, then (rows that do not fit the registers) [H] the row
    float* red = nan_row;
    float* row = nan_row + 32;
    pdl_trigger();
    const int r = blockIdx.x;
    pdl_wait();
    float* xr = stream + (size_t)r * H;
    const float* yr = y + (size_t)r * H;
    TO* orow = out2 + (size_t)r * H;
    if (!ZLM_CHK(xr, (size_t)H * 4) || !ZLM_CHK(yr, (size_t)H * 4) || !ZLM_CHK(orow, (size_t)H * sizeof(TO))) return;
    if (in_regs) {
        // H a multiple of 4 and up to NORM_MAX_V4 float4 a thread: the row is read once and stays in registers
        const int nv = H / 4;
        float4 v[NORM_MAX_V4], x[NORM_MAX_V4];
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < NORM_MAX_V4; ++j) {
            const int c = threadIdx.x + j * blockDim.x;
            v[j] = c < nv ? *(const float4*)(yr + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            x[j] = c < nv ? *(const float4*)(xr + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            s = fmaf(v[j].x, v[j].x, s); s = fmaf(v[j].y, v[j].y, s);
            s = fmaf(v[j].z, v[j].z, s); s = fmaf(v[j].w, v[j].w, s);
        }
        const float inv1 = 1.0f / sqrtf(block_sum(s, red) / (float)H + eps1);
        float s2 = 0.f;
#pragma unroll
        for (int j = 0; j < NORM_MAX_V4; ++j) {
            const int c = threadIdx.x + j * blockDim.x;
            if (c >= nv) continue;
            const float4 wv = w1.load4(c * 4);
            float4 a = x[j];
            a.x += (v[j].x * inv1) * wv.x; a.y += (v[j].y * inv1) * wv.y;
            a.z += (v[j].z * inv1) * wv.z; a.w += (v[j].w * inv1) * wv.w;
            *(float4*)(xr + c * 4) = a;
            v[j] = a;
            s2 = fmaf(a.x, a.x, s2); s2 = fmaf(a.y, a.y, s2); s2 = fmaf(a.z, a.z, s2); s2 = fmaf(a.w, a.w, s2);
        }
        const float inv2 = 1.0f / sqrtf(block_sum(s2, red) / (float)H + eps2);
#pragma unroll
        for (int j = 0; j < NORM_MAX_V4; ++j) {
            const int c = threadIdx.x + j * blockDim.x;
            if (c >= nv) continue;
            const float4 wv = w2.load4(c * 4);
            store4(orow + c * 4, (v[j].x * inv2) * wv.x, (v[j].y * inv2) * wv.y, (v[j].z * inv2) * wv.z, (v[j].w * inv2) * wv.w);
        }
        return;
    }
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float a = yr[i];
        row[i] = a;
        s = fmaf(a, a, s);
    }
    const float inv1 = 1.0f / sqrtf(block_sum(s, red) / (float)H + eps1);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float a = xr[i] + (row[i] * inv1) * w1[i];
        xr[i] = a;
        row[i] = a;
        s2 = fmaf(a, a, s2);
    }
    const float inv2 = 1.0f / sqrtf(block_sum(s2, red) / (float)H + eps2);
    for (int i = threadIdx.x; i < H; i += blockDim.x) orow[i] = from_f32<TO>((row[i] * inv2) * w2[i]);
}

extern "C" int zlm_norm_add_norm(float* stream, const float* y, const void* w1, int w1_dtype, float eps1, void* out2,
                                 int out2_dtype, const void* w2, int w2_dtype, float eps2, int R, int H, cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    ZLM_REQUIRE(R > 0 && H > 0 && H <= 11264, "norm_add_norm: bad sizes R=%d H=%d (rows of up to 11264)", R, H);
    int threads = 128;
    while (threads < 1024 && threads * 4 * NORM_MAX_V4 < H) threads *= 2;
    const int in_regs = (H % 4 == 0 && H / 4 <= NORM_MAX_V4 * threads && (uintptr_t)stream % 16 == 0 && (uintptr_t)y % 16 == 0 &&
                         (uintptr_t)w1 % 16 == 0 && (uintptr_t)w2 % 16 == 0 && (uintptr_t)out2 % 16 == 0) ? 1 : 0;
    const size_t smem = (size_t)(32 + (in_regs ? 0 : H)) * sizeof(float);
    const VecW v1{w1, w1_dtype}, v2{w2, w2_dtype};
    if (out2_dtype == ZLM_DTYPE_F32)
        zlm_launch(norm_add_norm_kernel<float>, R, threads, smem, st, stream, y, v1, eps1, (float*)out2, v2, eps2, H, in_regs);
    else if (out2_dtype == ZLM_DTYPE_BF16)
        zlm_launch(norm_add_norm_kernel<__nv_bfloat16>, R, threads, smem, st, stream, y, v1, eps1, (__nv_bfloat16*)out2, v2,
                   eps2, H, in_regs);
    else
        ZLM_REQUIRE(false, "norm_add_norm: unsupported output dtype %d", out2_dtype);
    return zlm_check_launch("norm_add_norm");
}

// ---------------------------------------------------------------- the stream's rows in the compute dtype
__global__ void cast_rows_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ x, size_t n4, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x; c < n4; c += (size_t)gridDim.x * blockDim.x) {
        if (!ZLM_CHK(x + c * 4, 16) || !ZLM_CHK(out + c * 4, 8)) continue;
        const float4 v = *(const float4*)(x + c * 4);
        store4(out + c * 4, v.x, v.y, v.z, v.w);
    }
    // a tail of up to three elements
    if (blockIdx.x == 0)
        for (size_t i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x)
            if (ZLM_CHK(x + i, 4) && ZLM_CHK(out + i, 2)) out[i] = __float2bfloat16_rn(x[i]);
}

extern "C" int zlm_cast_rows(void* out, const float* x, long long n, cudaStream_t st) {
    if (n == 0) return ZLM_OK;
    ZLM_REQUIRE(n > 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 8 == 0, "cast_rows: %lld elements, aligned operands", n);
    const size_t n4 = (size_t)n / 4;
    long long blocks = (long long)((n4 + 255) / 256);
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    zlm_launch(cast_rows_kernel, (int)blocks, 256, 0, st, (__nv_bfloat16*)out, x, n4, (size_t)n);
    return zlm_check_launch("cast_rows");
}

// ---------------------------------------------------------------- gated activation
__device__ __forceinline__ float zlm_gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// gu is [T, 2I]: gate in columns [0, I), up in [I, 2I); act 0: silu, 1: the tanh form of gelu
template <typename TA>
__global__ void gated_act_kernel(TA* __restrict__ out, const TA* __restrict__ gu, int T, int I, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)T * I;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / I;
        const int i = (int)(e - t * I);
        if (!ZLM_CHK(&gu[t * 2 * I + i], sizeof(TA)) || !ZLM_CHK(&gu[t * 2 * I + I + i], sizeof(TA)) ||
            !ZLM_CHK(&out[e], sizeof(TA)))
            continue;
        const float g = to_f32(gu[t * 2 * I + i]);
        const float u = to_f32(gu[t * 2 * I + I + i]);
        const float a = act == 1 ? zlm_gelu_tanh(g) : g / (1.0f + expf(-g));
        out[e] = from_f32<TA>(a * u);
    }
}

extern "C" int zlm_gated_act(void* out, const void* gu, int dtype, int T, int I, int act, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && I > 0 && (act == 0 || act == 1), "gated_act: bad sizes T=%d I=%d act=%d", T, I, act);
    const size_t n = (size_t)T * I;
    int blocks = (int)((n + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(gated_act_kernel<float>, blocks, 256, 0, st, (float*)out, (const float*)gu, T, I, act);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(gated_act_kernel<__nv_bfloat16>, blocks, 256, 0, st, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, T, I, act);
    else
        ZLM_REQUIRE(false, "gated_act: unsupported dtype %d", dtype);
    return zlm_check_launch("gated_act");
}

// ---------------------------------------------------------------- x *= s
__global__ void scale_f32_kernel(float* __restrict__ x, size_t n, float s) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        if (ZLM_CHK(x + i, 4)) x[i] *= s;
}

extern "C" int zlm_scale_f32(float* x, long long n, float s, cudaStream_t st) {
    if (n <= 0) return ZLM_OK;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    zlm_launch(scale_f32_kernel, (int)blocks, 256, 0, st, x, (size_t)n, s);
    return zlm_check_launch("scale_f32");
}

// ---------------------------------------------------------------- out (+)= alpha a + beta b
// The sum of two sublayers that ran side by side on one input, each with a scale of its own; fp32.
__global__ void scaled_sum_kernel(float* __restrict__ out, const float* __restrict__ a, float alpha, const float* __restrict__ b,
                                  float beta, size_t n, int accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        if (!ZLM_CHK(out + i, 4) || !ZLM_CHK(a + i, 4) || !ZLM_CHK(b + i, 4)) continue;
        const float y = fmaf(alpha, a[i], beta * b[i]);
        out[i] = accumulate ? out[i] + y : y;
    }
}

extern "C" int zlm_scaled_sum(float* out, const float* a, float alpha, const float* b, float beta, long long n, int accumulate,
                              cudaStream_t st) {
    if (n <= 0) return ZLM_OK;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    zlm_launch(scaled_sum_kernel, (int)blocks, 256, 0, st, out, a, alpha, b, beta, (size_t)n, accumulate);
    return zlm_check_launch("scaled_sum");
}

// ---------------------------------------------------------------- x = cap * tanh(x / cap)
__global__ void softcap_f32_kernel(float* __restrict__ x, size_t n, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        if (ZLM_CHK(x + i, 4)) x[i] = cap * tanhf(x[i] / cap);
}

extern "C" int zlm_softcap_f32(float* x, long long n, float cap, cudaStream_t st) {
    if (n <= 0) return ZLM_OK;
    ZLM_REQUIRE(cap > 0.f, "softcap: cap %g", (double)cap);
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    zlm_launch(softcap_f32_kernel, (int)blocks, 256, 0, st, x, (size_t)n, cap);
    return zlm_check_launch("softcap_f32");
}

// ---------------------------------------------------------------- silu in place on the first columns of every row
template <typename TA>
__global__ void silu_rows_kernel(TA* __restrict__ x, int stride, int T, int cols) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)T * cols;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / cols;
        TA* p = x + t * stride + (e - t * cols);
        if (!ZLM_CHK(p, sizeof(TA))) continue;
        const float z = to_f32(*p);
        *p = from_f32<TA>(z / (1.0f + expf(-z)));
    }
}

extern "C" int zlm_silu_rows(void* x, int stride, int dtype, int T, int cols, cudaStream_t st) {
    if (T <= 0 || cols <= 0) return ZLM_OK;
    ZLM_REQUIRE(stride >= cols, "silu_rows: %d columns in rows of %d", cols, stride);
    const size_t n = (size_t)T * cols;
    int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(silu_rows_kernel<float>, blocks, 256, 0, st, (float*)x, stride, T, cols);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(silu_rows_kernel<__nv_bfloat16>, blocks, 256, 0, st, (__nv_bfloat16*)x, stride, T, cols);
    else
        ZLM_REQUIRE(false, "silu_rows: unsupported dtype %d", dtype);
    return zlm_check_launch("silu_rows");
}

// ---------------------------------------------------------------- gated activation with clamped operands
// out = g' * sigmoid(alpha g') * (u' + 1), g' = min(gate, limit), u' = clamp(up, -limit, limit); gu is [T, 2I]: gate in
// columns [0, I), up in [I, 2I)
template <typename TA>
__global__ void gated_limit_kernel(TA* __restrict__ out, const TA* __restrict__ gu, int T, int I, float limit, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)T * I;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / I;
        const int i = (int)(e - t * I);
        if (!ZLM_CHK(&gu[t * 2 * I + i], sizeof(TA)) || !ZLM_CHK(&gu[t * 2 * I + I + i], sizeof(TA)) ||
            !ZLM_CHK(&out[e], sizeof(TA)))
            continue;
        const float g = fminf(to_f32(gu[t * 2 * I + i]), limit);
        const float u = fminf(fmaxf(to_f32(gu[t * 2 * I + I + i]), -limit), limit);
        out[e] = from_f32<TA>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}

extern "C" int zlm_gated_limit(void* out, const void* gu, int dtype, int T, int I, float limit, float alpha, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && I > 0 && limit > 0.f, "gated_limit: bad sizes T=%d I=%d limit=%g", T, I, (double)limit);
    const size_t n = (size_t)T * I;
    int blocks = (int)((n + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(gated_limit_kernel<float>, blocks, 256, 0, st, (float*)out, (const float*)gu, T, I, limit, alpha);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(gated_limit_kernel<__nv_bfloat16>, blocks, 256, 0, st, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, T, I,
                   limit, alpha);
    else
        ZLM_REQUIRE(false, "gated_limit: unsupported dtype %d", dtype);
    return zlm_check_launch("gated_limit");
}

// ---------------------------------------------------------------- one gate number per head
// x [T, heads, V] (any token and head strides) *= sigmoid(g[t, h]); a warp per (token, head)
template <typename TA>
__global__ void head_scalar_gate_kernel(TA* __restrict__ x, int x_stride, int x_hstride, const TA* __restrict__ g,
                                        int g_stride, int T, int H, int V) {
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)T * H) return;
    const int t = (int)(unit / H), h = (int)(unit % H);
    pdl_wait();
    TA* xp = x + (size_t)t * x_stride + (size_t)h * x_hstride;
    const TA* gp = g + (size_t)t * g_stride + h;
    if (!ZLM_CHK(xp, (size_t)V * sizeof(TA)) || !ZLM_CHK(gp, sizeof(TA))) return;
    const float gate = 1.0f / (1.0f + expf(-to_f32(*gp)));
    for (int e = lane; e < V; e += 32) xp[e] = from_f32<TA>(to_f32(xp[e]) * gate);
}

extern "C" int zlm_head_scalar_gate(void* x, int x_stride, int x_hstride, const void* g, int g_stride, int dtype, int T,
                                    int H, int V, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(H > 0 && V > 0, "head_scalar_gate: %d heads of %d", H, V);
    const long long units = (long long)T * H;
    const int blocks = (int)((units + 3) / 4);
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(head_scalar_gate_kernel<float>, blocks, 128, 0, st, (float*)x, x_stride, x_hstride, (const float*)g,
                   g_stride, T, H, V);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(head_scalar_gate_kernel<__nv_bfloat16>, blocks, 128, 0, st, (__nv_bfloat16*)x, x_stride, x_hstride,
                   (const __nv_bfloat16*)g, g_stride, T, H, V);
    else
        ZLM_REQUIRE(false, "head_scalar_gate: unsupported dtype %d", dtype);
    return zlm_check_launch("head_scalar_gate");
}

ZLM_TRANSLATION_UNIT(stream_ops)
