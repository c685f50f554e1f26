// A short causal convolution over time on every channel of a fused q/k/v projection, and what follows it in
// an attention mixer that has one: per-head unit RMS norm of q and k (no weight), q written out head by head,
// k and v written to the token's place in the paged cache.  The counterpart, for such a mixer, of the
// norm / rotation / cache-write kernel of the rotary attention mixer.
//
//   y_t[c] = sum_j w[c][j] * u_(t - taps + 1 + j)[c],  j = 0 .. taps-1,  zeros before the sequence's start
//
// u are the projected values.  Those of the step's own earlier tokens are read from the projection buffer
// (a sequence's tokens are neighbours in a step); those of earlier steps come from the sequence's state,
// [slots][taps-1][channels], whose row taps-2 is the newest.  A second kernel writes the state's new rows
// after the step (a thread owns one channel of one sequence: it reads all it needs before it writes).
//
// Heads are padded to `hdp` columns (zeros) in q_out and in the cache, so that keys of `dim` and values of
// `vdim` columns share the attention kernels' [K|V][kv head][token][hdp] page layout.
// Sums (taps, squares) are fp32 in both element types.
#include "common.cuh"

#define SC_WARPS 4
#define SC_MAX_TAPS 8
#define SC_MAX_PER_LANE 16      // head sizes up to 512

// VEC consecutive elements as floats, and back (VEC 4: one 8- or 16-byte access; the caller has checked the alignment)
template <typename TA, int VEC>
__device__ __forceinline__ void load_vec(const TA* __restrict__ p, float* f) {
    if (VEC == 1) {
        f[0] = to_f32(p[0]);
    } else if (sizeof(TA) == 2) {
        const uint2 u = *(const uint2*)p;
        f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
        f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
    } else {
        const float4 v = *(const float4*)p;
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
}
template <typename TA, int VEC>
__device__ __forceinline__ void store_vec(TA* __restrict__ p, const float* f) {
    if (VEC == 1) {
        p[0] = from_f32<TA>(f[0]);
    } else if (sizeof(TA) == 2) {
        __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
        uint2 u;
        u.x = *(unsigned*)&a; u.y = *(unsigned*)&b;
        *(uint2*)p = u;
    } else {
        *(float4*)p = make_float4(f[0], f[1], f[2], f[3]);
    }
}

// a warp per head (q, k or v) of one token; a lane owns VEC neighbouring channels at a time
template <typename TA, int VEC>
__global__ void __launch_bounds__(SC_WARPS * 32)
conv_norm_write_kernel(TA* __restrict__ q_out, int q_out_stride, const TA* __restrict__ proj, int proj_stride,
                       const TA* __restrict__ conv_w, const TA* __restrict__ state, const int* __restrict__ token_pos,
                       const int* __restrict__ token_slot, const int* __restrict__ token_seq,
                       const int* __restrict__ seq_start, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ block_table, int table_stride, TA* __restrict__ pool, int nq, int nkv,
                       int dim, int vdim, int hdp, int taps, int norm, float eps) {
    constexpr int ITER = SC_MAX_PER_LANE / VEC;
    pdl_trigger();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int unit = blockIdx.y * SC_WARPS + warp;
    if (unit >= nq + 2 * nkv) return;
    pdl_wait();
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(token_slot + t, 4) || !ZLM_CHK(token_seq + t, 4)) return;
    const int pos = token_pos[t], slot = token_slot[t], r = token_seq[t];
    if (!ZLM_CHK(seq_start + r, 4) || !ZLM_CHK(cu_seqlens + r, 4)) return;
    const int i = pos - seq_start[r];             // the token's place among its sequence's tokens of this step
    const int row0 = cu_seqlens[r];
    const int C = (nq + nkv) * dim + nkv * vdim;
    const int kind = unit < nq ? 0 : (unit < nq + nkv ? 1 : 2);
    const int width = kind == 2 ? vdim : dim;
    const int c0 = kind == 0 ? unit * dim : (kind == 1 ? nq * dim + (unit - nq) * dim : (nq + nkv) * dim + (unit - nq - nkv) * vdim);

    float val[ITER][VEC];
    float ss = 0.f;
#pragma unroll
    for (int rr = 0; rr < ITER; ++rr) {
        const int e = (lane + 32 * rr) * VEC;
#pragma unroll
        for (int v = 0; v < VEC; ++v) val[rr][v] = 0.f;
        if (e >= width) continue;
        const int c = c0 + e;
        for (int j = 0; j < taps; ++j) {
            const int s = i - (taps - 1) + j;
            if (pos - (taps - 1) + j < 0) continue;                       // before the sequence's start
            const TA* up = s >= 0 ? proj + (size_t)(row0 + s) * proj_stride + c
                                  : state + ((size_t)slot * (taps - 1) + (taps - 1 + s)) * C + c;
            if (!ZLM_CHK(up, VEC * sizeof(TA)) || !ZLM_CHK(conv_w + (size_t)c * taps, (size_t)VEC * taps * sizeof(TA))) continue;
            float u[VEC];
            load_vec<TA, VEC>(up, u);
#pragma unroll
            for (int v = 0; v < VEC; ++v) val[rr][v] = fmaf(to_f32(conv_w[(size_t)(c + v) * taps + j]), u[v], val[rr][v]);
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) ss = fmaf(val[rr][v], val[rr][v], ss);
    }
    float scale = 1.0f;
    if (norm && kind != 2) {
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)width + eps);
    }
    TA* dst;
    if (kind == 0) {
        dst = q_out + (size_t)t * q_out_stride + (size_t)unit * hdp;
    } else {
        if (!ZLM_CHK(block_table + (size_t)slot * table_stride + pos / ZLM_PAGE, 4)) return;
        const int page = block_table[(size_t)slot * table_stride + pos / ZLM_PAGE];
        const int kvh = kind == 1 ? unit - nq : unit - nq - nkv;
        dst = pool + (((size_t)page * 2 + (kind - 1)) * nkv + kvh) * ZLM_PAGE * hdp + (size_t)(pos % ZLM_PAGE) * hdp;
    }
    if (!ZLM_CHK(dst, (size_t)hdp * sizeof(TA))) return;
#pragma unroll
    for (int rr = 0; rr < ITER; ++rr) {
        const int e = (lane + 32 * rr) * VEC;
        if (e >= hdp) continue;
        float o[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) o[v] = e + v < width ? val[rr][v] * scale : 0.f;       // (width and hdp are multiples of VEC)
        store_vec<TA, VEC>(dst + e, o);
    }
}

// state[slot][m] <- the (taps-1) newest projected values of the sequence after this step, m = taps-2 the newest
template <typename TA>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(TA* __restrict__ state, const TA* __restrict__ proj, int proj_stride,
                         const int* __restrict__ seq_slot, const int* __restrict__ cu_seqlens, int C, int taps) {
    pdl_trigger();
    const int r = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    pdl_wait();
    if (c >= C || !ZLM_CHK(seq_slot + r, 4) || !ZLM_CHK(cu_seqlens + r, 8)) return;
    const int slot = seq_slot[r], row0 = cu_seqlens[r], n = cu_seqlens[r + 1] - row0;
    TA keep[SC_MAX_TAPS];
    for (int m = 0; m < taps - 1; ++m) {
        const int s = n - (taps - 1) + m;
        const TA* up = s >= 0 ? proj + (size_t)(row0 + s) * proj_stride + c
                              : state + ((size_t)slot * (taps - 1) + (taps - 1 + s)) * C + c;
        keep[m] = ZLM_CHK(up, sizeof(TA)) ? *up : from_f32<TA>(0.f);
    }
    for (int m = 0; m < taps - 1; ++m) {
        TA* p = state + ((size_t)slot * (taps - 1) + m) * C + c;
        if (ZLM_CHK(p, sizeof(TA))) *p = keep[m];
    }
}

template <typename TA>
static void launch_conv(void* q_out, int q_out_stride, const void* proj, int proj_stride, const void* conv_w, void* state,
                        const int* token_pos, const int* token_slot, const int* token_seq, const int* seq_start,
                        const int* cu_seqlens, const int* seq_slot, const int* block_table, int table_stride, void* pool,
                        int T, int R, int nq, int nkv, int dim, int vdim, int hdp, int taps, int norm, float eps,
                        cudaStream_t st) {
    const int units = nq + 2 * nkv;
    const int C0 = (nq + nkv) * dim + nkv * vdim;
    // four neighbouring channels a lane where every row and head starts at a multiple of four elements, 8 or 16 bytes
    const size_t al = 4 * sizeof(TA);
    const bool vec = dim % 4 == 0 && vdim % 4 == 0 && hdp % 4 == 0 && proj_stride % 4 == 0 && q_out_stride % 4 == 0 && C0 % 4 == 0 &&
                     (uintptr_t)proj % al == 0 && (uintptr_t)q_out % al == 0 && (uintptr_t)pool % al == 0 &&
                     (state == nullptr || (uintptr_t)state % al == 0);
    if (vec)
        zlm_launch(conv_norm_write_kernel<TA, 4>, dim3(T, (units + SC_WARPS - 1) / SC_WARPS), dim3(SC_WARPS * 32), 0, st,
                   (TA*)q_out, q_out_stride, (const TA*)proj, proj_stride, (const TA*)conv_w, (const TA*)state, token_pos,
                   token_slot, token_seq, seq_start, cu_seqlens, block_table, table_stride, (TA*)pool, nq, nkv, dim, vdim, hdp,
                   taps, norm, eps);
    else
        zlm_launch(conv_norm_write_kernel<TA, 1>, dim3(T, (units + SC_WARPS - 1) / SC_WARPS), dim3(SC_WARPS * 32), 0, st,
                   (TA*)q_out, q_out_stride, (const TA*)proj, proj_stride, (const TA*)conv_w, (const TA*)state, token_pos,
                   token_slot, token_seq, seq_start, cu_seqlens, block_table, table_stride, (TA*)pool, nq, nkv, dim, vdim, hdp,
                   taps, norm, eps);
    if (taps > 1) {
        const int C = (nq + nkv) * dim + nkv * vdim;
        zlm_launch(conv_state_update_kernel<TA>, dim3(R, (C + 255) / 256), dim3(256), 0, st, (TA*)state, (const TA*)proj,
                   proj_stride, seq_slot, cu_seqlens, C, taps);
    }
}

// proj [T][proj_stride]: columns [q: nq*dim | k: nkv*dim | v: nkv*vdim | anything]; conv_w [channels][taps] in the same
// element type; state [slots][taps-1][channels] (unused if taps == 1); q_out [T][q_out_stride] receives nq heads of hdp
// columns; pool [pages][2][nkv][64][hdp].  norm: q and k heads are divided by their root mean square over dim.
extern "C" int zlm_conv_norm_write(void* q_out, int q_out_stride, const void* proj, int proj_stride, const void* conv_w,
                                   void* state, int dtype, const int* token_pos, const int* token_slot,
                                   const int* token_seq, const int* seq_start, const int* cu_seqlens, const int* seq_slot,
                                   const int* block_table, int table_stride, void* pool, int T, int R, int nq, int nkv,
                                   int dim, int vdim, int hdp, int taps, int norm, float eps, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(nq > 0 && nkv > 0 && dim > 0 && vdim > 0 && hdp >= dim && hdp >= vdim && hdp <= 32 * SC_MAX_PER_LANE,
                "conv_norm_write: heads %d/%d of %d and %d columns padded to %d (at most %d)", nq, nkv, dim, vdim, hdp,
                32 * SC_MAX_PER_LANE);
    ZLM_REQUIRE(taps >= 1 && taps <= SC_MAX_TAPS, "conv_norm_write: %d taps (at most %d)", taps, SC_MAX_TAPS);
    ZLM_REQUIRE(taps == 1 || state, "conv_norm_write: a convolution of %d taps needs the sequences' state", taps);
    ZLM_REQUIRE(T <= 2147483647 / 2 && R <= 65535 * 1024 && (nq + 2 * nkv + SC_WARPS - 1) / SC_WARPS <= 65535,
                "conv_norm_write: too many tokens, sequences or heads");
    if (dtype == ZLM_DTYPE_F32)
        launch_conv<float>(q_out, q_out_stride, proj, proj_stride, conv_w, state, token_pos, token_slot, token_seq, seq_start,
                           cu_seqlens, seq_slot, block_table, table_stride, pool, T, R, nq, nkv, dim, vdim, hdp, taps, norm,
                           eps, st);
    else if (dtype == ZLM_DTYPE_BF16)
        launch_conv<__nv_bfloat16>(q_out, q_out_stride, proj, proj_stride, conv_w, state, token_pos, token_slot, token_seq,
                                   seq_start, cu_seqlens, seq_slot, block_table, table_stride, pool, T, R, nq, nkv, dim, vdim,
                                   hdp, taps, norm, eps, st);
    else
        ZLM_REQUIRE(false, "conv_norm_write: unsupported dtype %d", dtype);
    return zlm_check_launch("conv_norm_write");
}

// ---------------------------------------------------------------------------- heads times a gate
// out[t][h*V + e] = unit_norm?(o[t][h][:V])[e] * act(g[t][h*V + e]): the heads of a mixer's output, each optionally
// divided by its root mean square (fp32), times sigmoid (act 0) or silu (act 1) of a gate projection, written
// without the heads' padding.  o may be fp32 whatever the element type (a recurrence's output).
template <typename TO, typename TA, int VEC>
__global__ void __launch_bounds__(SC_WARPS * 32)
head_gate_kernel(TA* __restrict__ out, int out_stride, const TO* __restrict__ o, int o_stride, int o_head_stride,
                 const TA* __restrict__ g, int g_stride, int H, int V, int norm, float eps, int act) {
    constexpr int ITER = SC_MAX_PER_LANE / VEC;
    pdl_trigger();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * SC_WARPS + warp;
    if (h >= H) return;
    pdl_wait();
    const TO* op = o + (size_t)t * o_stride + (size_t)h * o_head_stride;
    const TA* gp = g + (size_t)t * g_stride + (size_t)h * V;
    TA* dst = out + (size_t)t * out_stride + (size_t)h * V;
    if (!ZLM_CHK(op, (size_t)V * sizeof(TO)) || !ZLM_CHK(gp, (size_t)V * sizeof(TA)) || !ZLM_CHK(dst, (size_t)V * sizeof(TA)))
        return;
    float val[ITER][VEC];
    float ss = 0.f;
#pragma unroll
    for (int rr = 0; rr < ITER; ++rr) {
        const int e = (lane + 32 * rr) * VEC;
#pragma unroll
        for (int v = 0; v < VEC; ++v) val[rr][v] = 0.f;
        if (e >= V) continue;
        load_vec<TO, VEC>(op + e, val[rr]);
#pragma unroll
        for (int v = 0; v < VEC; ++v) ss = fmaf(val[rr][v], val[rr][v], ss);
    }
    float scale = 1.0f;
    if (norm) scale = 1.0f / sqrtf(warp_sum(ss) / (float)V + eps);
#pragma unroll
    for (int rr = 0; rr < ITER; ++rr) {
        const int e = (lane + 32 * rr) * VEC;
        if (e >= V) continue;
        float z[VEC], y[VEC];
        load_vec<TA, VEC>(gp + e, z);
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const float sg = 1.0f / (1.0f + expf(-z[v]));
            y[v] = val[rr][v] * scale * (act == 1 ? z[v] * sg : sg);
        }
        store_vec<TA, VEC>(dst + e, y);
    }
}

extern "C" int zlm_head_gate(void* out, int out_stride, const void* o, int o_is_f32, int o_stride, int o_head_stride,
                             const void* g, int g_stride, int dtype, int T, int H, int V, int norm, float eps, int act,
                             cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(H > 0 && V > 0 && V <= 32 * SC_MAX_PER_LANE && (H + SC_WARPS - 1) / SC_WARPS <= 65535,
                "head_gate: %d heads of %d columns (at most %d)", H, V, 32 * SC_MAX_PER_LANE);
    ZLM_REQUIRE(act == 0 || act == 1, "head_gate: activation %d", act);
    const dim3 grid(T, (H + SC_WARPS - 1) / SC_WARPS), block(SC_WARPS * 32);
    // four neighbouring columns a lane where every row and head starts at a multiple of 16 bytes
    const bool vec = V % 4 == 0 && out_stride % 4 == 0 && o_stride % 4 == 0 && o_head_stride % 4 == 0 && g_stride % 4 == 0 &&
                     (uintptr_t)out % 16 == 0 && (uintptr_t)o % 16 == 0 && (uintptr_t)g % 16 == 0;
#define ZLM_HG(TO, TA, VEC)                                                                                              \
    zlm_launch(head_gate_kernel<TO, TA, VEC>, grid, block, 0, st, (TA*)out, out_stride, (const TO*)o, o_stride, o_head_stride, \
               (const TA*)g, g_stride, H, V, norm, eps, act)
    if (dtype == ZLM_DTYPE_F32) {
        if (vec) ZLM_HG(float, float, 4); else ZLM_HG(float, float, 1);
    } else if (dtype == ZLM_DTYPE_BF16 && o_is_f32) {
        if (vec) ZLM_HG(float, __nv_bfloat16, 4); else ZLM_HG(float, __nv_bfloat16, 1);
    } else if (dtype == ZLM_DTYPE_BF16) {
        if (vec) ZLM_HG(__nv_bfloat16, __nv_bfloat16, 4); else ZLM_HG(__nv_bfloat16, __nv_bfloat16, 1);
    } else {
        ZLM_REQUIRE(false, "head_gate: unsupported dtype %d", dtype);
    }
#undef ZLM_HG
    return zlm_check_launch("head_gate");
}


// ---------------------------------------------------------------------------- q/k/v preparation, general form
// What stands between a fused q/k/v projection and attention over the paged cache, with every step optional:
//   a short causal convolution per channel (as above; has_conv 0: none),
//   a norm of q and k: per head without weight (norm_mode 1), per head with one weight of `dim` shared by the heads
//   (2), or over the whole projection at once, all heads of q (of k) together, with a weight per channel (3),
//   rotation of the first n_rot coordinates of every q and k head, coordinate i against i + n_rot/2, by the angle
//   pos * inv_freq[i]; cosine and sine are multiplied by rot_scale (a frequency table scaled for long contexts
//   carries such a factor),
//   q written head by head, k and v into the token's place of the paged cache, heads padded with zeros to hdp.
// A block per token: the token's convolved channels are held in shared memory as fp32, the sums of squares are
// block sums in a fixed order, angles, cosines and sines are fp32.
#define AP_THREADS 256
template <typename TA>
__global__ void __launch_bounds__(AP_THREADS)
attn_prep_kernel(TA* __restrict__ q_out, int q_out_stride, const TA* __restrict__ proj, int proj_stride,
                 const TA* __restrict__ conv_w, const TA* __restrict__ state, const int* __restrict__ token_pos,
                 const int* __restrict__ token_slot, const int* __restrict__ token_seq, const int* __restrict__ seq_start,
                 const int* __restrict__ cu_seqlens, const int* __restrict__ block_table, int table_stride,
                 TA* __restrict__ pool, int nq, int nkv, int dim, int vdim, int hdp, int taps, int norm_mode, VecW q_w,
                 VecW k_w, float eps, const float* __restrict__ inv_freq, int n_rot, float rot_scale) {
    extern __shared__ float ap_smem[];          // [C] channels, [nq + nkv] inverse root mean squares, [32] reduction
    pdl_trigger();
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int QC = nq * dim, KC = nkv * dim, C = QC + KC + nkv * vdim;
    float* val = ap_smem;
    float* inv = ap_smem + C;
    float* red = inv + nq + nkv;
    float* rot = red + 32;                      // [n_rot/2] cosines, [n_rot/2] sines of the token's angles
    pdl_wait();
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(token_slot + t, 4) || !ZLM_CHK(token_seq + t, 4)) return;
    const int pos = token_pos[t], slot = token_slot[t], r = token_seq[t];
    if (!ZLM_CHK(seq_start + r, 4) || !ZLM_CHK(cu_seqlens + r, 4)) return;
    const int i = pos - seq_start[r];
    const int row0 = cu_seqlens[r];
    float ssq = 0.f, ssk = 0.f;
    for (int c = tid; c < C; c += AP_THREADS) {
        float a = 0.f;
        if (conv_w) {
            for (int j = 0; j < taps; ++j) {
                const int s = i - (taps - 1) + j;
                if (pos - (taps - 1) + j < 0) continue;
                const TA* up = s >= 0 ? proj + (size_t)(row0 + s) * proj_stride + c
                                      : state + ((size_t)slot * (taps - 1) + (taps - 1 + s)) * C + c;
                if (!ZLM_CHK(up, sizeof(TA)) || !ZLM_CHK(conv_w + (size_t)c * taps + j, sizeof(TA))) continue;
                a = fmaf(to_f32(conv_w[(size_t)c * taps + j]), to_f32(*up), a);
            }
        } else {
            const TA* up = proj + (size_t)(row0 + i) * proj_stride + c;
            if (ZLM_CHK(up, sizeof(TA))) a = to_f32(*up);
        }
        val[c] = a;
        if (c < QC) ssq = fmaf(a, a, ssq); else if (c < QC + KC) ssk = fmaf(a, a, ssk);
    }
    __syncthreads();
    if (norm_mode == 3) {
        const float tq = block_sum(ssq, red);
        const float tk = block_sum(ssk, red);
        if (tid == 0) {
            const float iq = 1.0f / sqrtf(tq / (float)QC + eps), ik = 1.0f / sqrtf(tk / (float)KC + eps);
            for (int h = 0; h < nq; ++h) inv[h] = iq;
            for (int h = 0; h < nkv; ++h) inv[nq + h] = ik;
        }
    } else {
        for (int h = warp; h < nq + nkv; h += AP_THREADS / 32) {
            float ss = 0.f;
            for (int e = lane; e < dim; e += 32) { const float a = val[h * dim + e]; ss = fmaf(a, a, ss); }
            ss = warp_sum(ss);
            if (lane == 0) inv[h] = norm_mode ? 1.0f / sqrtf(ss / (float)dim + eps) : 1.0f;
        }
    }
    // the token's angles once a block: fp32 angle, sine and cosine, times the table's factor
    const int half = n_rot / 2;
    for (int f = tid; f < half; f += AP_THREADS) {
        float sn, cs;
        sincosf((float)pos * inv_freq[f], &sn, &cs);
        rot[f] = cs * rot_scale;
        rot[half + f] = sn * rot_scale;
    }
    __syncthreads();
    // q and k heads: norm, weight, rotation, write
    int page = 0;
    if (ZLM_CHK(block_table + (size_t)slot * table_stride + pos / ZLM_PAGE, 4))
        page = block_table[(size_t)slot * table_stride + pos / ZLM_PAGE];
    // (steps of few tokens run several blocks a token: each repeats the sums above and writes its share)
    for (int x = blockIdx.y * AP_THREADS + tid; x < (nq + 2 * nkv) * hdp; x += AP_THREADS * gridDim.y) {
        const int unit = x / hdp, e = x - unit * hdp;
        float o = 0.f;
        if (unit < nq + nkv) {
            if (e < dim) {
                const int c = unit * dim + e;
                const VecW& w = unit < nq ? q_w : k_w;
                const int wb = norm_mode == 3 ? (unit < nq ? unit * dim : (unit - nq) * dim) : 0;
                const float sc = inv[unit];
                o = val[c] * sc * (norm_mode >= 2 ? w[wb + e] : 1.0f);
                if (e < n_rot) {
                    const int fi = e < half ? e : e - half;
                    const int pe = e < half ? e + half : e - half;
                    const float other = val[unit * dim + pe] * sc * (norm_mode >= 2 ? w[wb + pe] : 1.0f);
                    const float cs = rot[fi], sn = rot[half + fi];
                    o = e < half ? o * cs - other * sn : o * cs + other * sn;
                }
            }
        } else if (e < vdim) {
            o = val[QC + KC + (unit - nq - nkv) * vdim + e];
        }
        TA* dst;
        if (unit < nq) {
            dst = q_out + (size_t)t * q_out_stride + (size_t)unit * hdp + e;
        } else {
            const int kind = unit < nq + nkv ? 0 : 1;
            const int kvh = kind == 0 ? unit - nq : unit - nq - nkv;
            dst = pool + (((size_t)page * 2 + kind) * nkv + kvh) * ZLM_PAGE * hdp + (size_t)(pos % ZLM_PAGE) * hdp + e;
        }
        if (ZLM_CHK(dst, sizeof(TA))) *dst = from_f32<TA>(o);
    }
}

template <typename TA>
static void launch_attn_prep(void* q_out, int q_out_stride, const void* proj, int proj_stride, const void* conv_w, void* state,
                             const int* token_pos, const int* token_slot, const int* token_seq, const int* seq_start,
                             const int* cu_seqlens, const int* seq_slot, const int* block_table, int table_stride, void* pool,
                             int T, int R, int nq, int nkv, int dim, int vdim, int hdp, int taps, int norm_mode, VecW q_w,
                             VecW k_w, float eps, const float* inv_freq, int n_rot, float rot_scale, cudaStream_t st) {
    const int C = (nq + nkv) * dim + nkv * vdim;
    const size_t smem = (size_t)(C + nq + nkv + 32 + n_rot) * sizeof(float);
    // blocks a token: one where the tokens alone fill the device, else as many as give it two rounds of work
    int share = 1;
    const int outputs = (nq + 2 * nkv) * hdp;
    while (share < 16 && (long long)T * share < 296 && outputs > share * AP_THREADS * 2) share *= 2;
    zlm_launch(attn_prep_kernel<TA>, dim3(T, share), dim3(AP_THREADS), smem, st, (TA*)q_out, q_out_stride, (const TA*)proj,
               proj_stride, (const TA*)conv_w, (const TA*)state, token_pos, token_slot, token_seq, seq_start, cu_seqlens,
               block_table, table_stride, (TA*)pool, nq, nkv, dim, vdim, hdp, taps, norm_mode, q_w, k_w, eps, inv_freq, n_rot,
               rot_scale);
    if (conv_w && taps > 1)
        zlm_launch(conv_state_update_kernel<TA>, dim3(R, (C + 255) / 256), dim3(256), 0, st, (TA*)state, (const TA*)proj,
                   proj_stride, seq_slot, cu_seqlens, C, taps);
}

// As zlm_conv_norm_write, with: conv_w null for no convolution; norm_mode 0 none, 1 per head without weight, 2 per
// head with q_w / k_w [dim], 3 over all heads at once with q_w [nq*dim] / k_w [nkv*dim]; inv_freq [n_rot/2] fp32
// (n_rot 0: no rotation); rot_scale multiplies cosines and sines.
extern "C" int zlm_attn_prep(void* q_out, int q_out_stride, const void* proj, int proj_stride, const void* conv_w,
                             void* state, int dtype, const int* token_pos, const int* token_slot, const int* token_seq,
                             const int* seq_start, const int* cu_seqlens, const int* seq_slot, const int* block_table,
                             int table_stride, void* pool, int T, int R, int nq, int nkv, int dim, int vdim, int hdp,
                             int taps, int norm_mode, const void* q_w, const void* k_w, int w_dtype, float eps,
                             const float* inv_freq, int n_rot, float rot_scale, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(nq > 0 && nkv > 0 && dim > 0 && vdim > 0 && hdp >= dim && hdp >= vdim, "attn_prep: heads %d/%d of %d and %d columns padded to %d",
                nq, nkv, dim, vdim, hdp);
    ZLM_REQUIRE(taps >= 1 && taps <= SC_MAX_TAPS, "attn_prep: %d taps (at most %d)", taps, SC_MAX_TAPS);
    ZLM_REQUIRE(!conv_w || taps == 1 || state, "attn_prep: a convolution of %d taps needs the sequences' state", taps);
    ZLM_REQUIRE(norm_mode >= 0 && norm_mode <= 3 && (norm_mode < 2 || (q_w && k_w)), "attn_prep: norm mode %d", norm_mode);
    ZLM_REQUIRE(n_rot >= 0 && n_rot % 2 == 0 && n_rot <= dim && (n_rot == 0 || inv_freq), "attn_prep: rotation over %d of %d coordinates", n_rot, dim);
    const size_t smem = (size_t)((nq + nkv) * dim + nkv * vdim + nq + nkv + 32 + n_rot) * sizeof(float);
    ZLM_REQUIRE(smem <= 200 * 1024, "attn_prep: %zu bytes of channels a token", smem);
    const VecW qw{q_w, w_dtype}, kw{k_w, w_dtype};
    if (dtype == ZLM_DTYPE_F32) {
        static bool big[64] = {};
        if (smem > 48 * 1024 && !big[zlm_device_index()]) {
            cudaFuncSetAttribute(attn_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            big[zlm_device_index()] = true;
        }
        launch_attn_prep<float>(q_out, q_out_stride, proj, proj_stride, conv_w, state, token_pos, token_slot, token_seq, seq_start,
                                cu_seqlens, seq_slot, block_table, table_stride, pool, T, R, nq, nkv, dim, vdim, hdp, taps,
                                norm_mode, qw, kw, eps, inv_freq, n_rot, rot_scale, st);
    } else if (dtype == ZLM_DTYPE_BF16) {
        static bool big[64] = {};
        if (smem > 48 * 1024 && !big[zlm_device_index()]) {
            cudaFuncSetAttribute(attn_prep_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            big[zlm_device_index()] = true;
        }
        launch_attn_prep<__nv_bfloat16>(q_out, q_out_stride, proj, proj_stride, conv_w, state, token_pos, token_slot, token_seq,
                                        seq_start, cu_seqlens, seq_slot, block_table, table_stride, pool, T, R, nq, nkv, dim,
                                        vdim, hdp, taps, norm_mode, qw, kw, eps, inv_freq, n_rot, rot_scale, st);
    } else {
        ZLM_REQUIRE(false, "attn_prep: unsupported dtype %d", dtype);
    }
    return zlm_check_launch("attn_prep");
}

// ---------------------------------------------------------------------------- norm, weight, gate on a recurrence's output
// out[t][c] = o[t][c] * inv_rms(group of c) * w[...] * act(g[t][c]) * out_scale, o fp32 [T][H*V]:
//   group 0: no norm; 1: every head of V columns by itself; 2: the whole row (all heads together);
//   w: none, [V] shared by the heads (w_rows 0) or [H*V] (w_rows 1);  act 0 sigmoid, 1 silu, 2 no gate.
// A block per token; sums of squares fp32 in a fixed order.
#define NG_THREADS 256
template <typename TA>
__global__ void __launch_bounds__(NG_THREADS)
norm_gate_kernel(TA* __restrict__ out, int out_stride, const float* __restrict__ o, const TA* __restrict__ g, int g_stride,
                 int H, int V, int group, VecW w, int has_w, int w_rows, float eps, int act, float out_scale) {
    extern __shared__ float ng_smem[];          // [H] inverse root mean squares, [32] reduction
    pdl_trigger();
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int N = H * V;
    float* inv = ng_smem;
    float* red = ng_smem + H;
    pdl_wait();
    const float* op = o + (size_t)t * N;
    if (group == 2) {
        float ss = 0.f;
        for (int c = tid; c < N; c += NG_THREADS) if (ZLM_CHK(op + c, 4)) ss = fmaf(op[c], op[c], ss);
        const float tot = block_sum(ss, red);
        if (tid < H) inv[tid] = 0.f;
        __syncthreads();
        const float s = 1.0f / sqrtf(tot / (float)N + eps);
        for (int h = tid; h < H; h += NG_THREADS) inv[h] = s;
    } else {
        for (int h = warp; h < H; h += NG_THREADS / 32) {
            float ss = 0.f;
            for (int e = lane; e < V; e += 32) if (ZLM_CHK(op + h * V + e, 4)) { const float a = op[h * V + e]; ss = fmaf(a, a, ss); }
            ss = warp_sum(ss);
            if (lane == 0) inv[h] = group == 1 ? 1.0f / sqrtf(ss / (float)V + eps) : 1.0f;
        }
    }
    __syncthreads();
    for (int c = tid; c < N; c += NG_THREADS) {
        const int h = c / V;
        if (!ZLM_CHK(op + c, 4)) continue;
        float y = op[c] * inv[h];
        if (has_w) y *= w[w_rows ? c : c - h * V];
        if (act != 2) {
            const TA* gp = g + (size_t)t * g_stride + c;
            if (!ZLM_CHK(gp, sizeof(TA))) continue;
            const float z = to_f32(*gp);
            const float sg = 1.0f / (1.0f + expf(-z));
            y *= act == 1 ? z * sg : sg;
        }
        TA* dst = out + (size_t)t * out_stride + c;
        if (ZLM_CHK(dst, sizeof(TA))) *dst = from_f32<TA>(y * out_scale);
    }
}

extern "C" int zlm_norm_gate(void* out, int out_stride, const float* o, const void* g, int g_stride, int dtype, int T, int H,
                             int V, int group, const void* w, int w_dtype, int w_rows, float eps, int act, float out_scale,
                             cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(H > 0 && V > 0 && H <= 8192 && group >= 0 && group <= 2 && act >= 0 && act <= 2 && (act == 2 || g),
                "norm_gate: %d heads of %d columns, group %d, activation %d", H, V, group, act);
    const VecW vw{w, w_dtype};
    const size_t smem = (size_t)(H + 32) * sizeof(float);
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(norm_gate_kernel<float>, dim3(T), dim3(NG_THREADS), smem, st, (float*)out, out_stride, o, (const float*)g,
                   g_stride, H, V, group, vw, w ? 1 : 0, w_rows, eps, act, out_scale);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(norm_gate_kernel<__nv_bfloat16>, dim3(T), dim3(NG_THREADS), smem, st, (__nv_bfloat16*)out, out_stride, o,
                   (const __nv_bfloat16*)g, g_stride, H, V, group, vw, w ? 1 : 0, w_rows, eps, act, out_scale);
    else
        ZLM_REQUIRE(false, "norm_gate: unsupported dtype %d", dtype);
    return zlm_check_launch("norm_gate");
}

ZLM_TRANSLATION_UNIT(short_conv)
