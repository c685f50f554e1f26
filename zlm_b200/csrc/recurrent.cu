// Recurrent mixers whose state is carried from token to token in fp32:
//
//   * a real-gated linear recurrent unit (one number of state per channel) behind a short causal convolution:
//       u = conv(x + b_x) + b_c                      x, y: two projections of the mixer's input
//       r = sigmoid(A_r[b] u_b + c_r),  i = sigmoid(A_i[b] u_b + c_i)      block-diagonal: u in `blocks` equal parts
//       log a = -c * r * softplus(lam),  S_t = a S_(t-1) + sqrt(1 - a^2) * i * u,   out = S_t * gelu_tanh(y + b_y)
//   * linear attention with a decay per key channel and token (gated linear attention) or per head:
//       S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t            S [dim][v_dim] per head
//     and the kernel that makes alpha from a low-rank projection: alpha = sigmoid(W2 lo + b)^(1/tau).
//
// Everything after the projections (convolution sums, gates, decays and their logarithms, softplus, exponentials,
// the state, the read-out) is fp32 in both element types.  A sequence's state is [slots][...] fp32 and is read at
// a step's start and written at its end; nothing is special about a sequence's first token: its state is zero.
#include "common.cuh"

#define RC_MAX_TAPS 8

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ---------------------------------------------------------------------------- convolution of the x branch
// u[t][c] = sum_j w[c][j] * (x_(t-taps+1+j)[c] + bx[c]) + cb[c]; x of the step's earlier tokens from `proj`, of earlier
// steps from the state's rows 1 .. taps-1 (row taps-1 the newest; they hold x + bx), zeros before the start.
template <typename TA>
__global__ void __launch_bounds__(256)
rglru_conv_kernel(float* __restrict__ u, const TA* __restrict__ proj, int proj_stride, int x_off, const TA* __restrict__ bx,
                  const TA* __restrict__ conv_w, const TA* __restrict__ cb, const float* __restrict__ state,
                  const int* __restrict__ token_pos, const int* __restrict__ token_slot, const int* __restrict__ token_seq,
                  const int* __restrict__ seq_start, const int* __restrict__ cu_seqlens, int W, int taps) {
    pdl_trigger();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    pdl_wait();
    if (c >= W) return;
    if (!ZLM_CHK(token_pos + t, 4) || !ZLM_CHK(token_slot + t, 4) || !ZLM_CHK(token_seq + t, 4)) return;
    const int pos = token_pos[t], slot = token_slot[t], r = token_seq[t];
    if (!ZLM_CHK(seq_start + r, 4) || !ZLM_CHK(cu_seqlens + r, 4)) return;
    const int i = pos - seq_start[r], row0 = cu_seqlens[r];
    const float b = bx ? to_f32(bx[c]) : 0.f;
    float a = cb ? to_f32(cb[c]) : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int s = i - (taps - 1) + j;
        if (pos - (taps - 1) + j < 0) continue;
        float x;
        if (s >= 0) {
            const TA* p = proj + (size_t)(row0 + s) * proj_stride + x_off + c;
            if (!ZLM_CHK(p, sizeof(TA))) continue;
            x = to_f32(*p) + b;
        } else {
            const float* p = state + ((size_t)slot * taps + (taps + s)) * W + c;
            if (!ZLM_CHK(p, 4)) continue;
            x = *p;
        }
        a = fmaf(to_f32(conv_w[(size_t)c * taps + j]), x, a);
    }
    if (ZLM_CHK(u + (size_t)t * W + c, 4)) u[(size_t)t * W + c] = a;
}

// ---------------------------------------------------------------------------- block-diagonal gate logits
// z[g][t][b*bs + o] = sum_i A_g[b][o][i] u[t][b*bs + i] + c_g[b*bs + o], g = 0 (recurrence gate), 1 (input gate).
// A block: 16 tokens x 64 outputs of one diagonal block, both gates; u and the weights in tiles of 32 inputs in shared
// memory; fp32 multiply-adds in a fixed order.
#define RG_TT 16
#define RG_OT 64
#define RG_KT 32
template <typename TA>
__global__ void __launch_bounds__(RG_OT * 4)
rglru_gates_kernel(float* __restrict__ zr, float* __restrict__ zi, const float* __restrict__ u, const TA* __restrict__ Ar,
                   const TA* __restrict__ Ai, const TA* __restrict__ cr, const TA* __restrict__ ci, int T, int W, int bs) {
    __shared__ float su[RG_TT][RG_KT + 1];
    __shared__ float sw[2][RG_OT][RG_KT + 1];
    pdl_trigger();
    const int t0 = blockIdx.x * RG_TT, b = blockIdx.z, o0 = blockIdx.y * RG_OT;
    const int tid = threadIdx.x, ol = tid % RG_OT, tq = tid / RG_OT;          // the thread's output, and its quarter of the tokens
    pdl_wait();
    float acc[2][RG_TT / 4];
#pragma unroll
    for (int g = 0; g < 2; ++g)
#pragma unroll
        for (int j = 0; j < RG_TT / 4; ++j) acc[g][j] = 0.f;
    for (int k0 = 0; k0 < bs; k0 += RG_KT) {
        for (int x = tid; x < RG_TT * RG_KT; x += RG_OT * 4) {
            const int tt = x / RG_KT, kk = x % RG_KT;
            const float* p = u + (size_t)(t0 + tt) * W + b * bs + k0 + kk;
            su[tt][kk] = (t0 + tt < T && k0 + kk < bs && ZLM_CHK(p, 4)) ? *p : 0.f;
        }
        for (int x = tid; x < 2 * RG_OT * RG_KT; x += RG_OT * 4) {
            const int g = x / (RG_OT * RG_KT), oo = (x / RG_KT) % RG_OT, kk = x % RG_KT;
            const TA* p = (g ? Ai : Ar) + ((size_t)b * bs + o0 + oo) * bs + k0 + kk;
            sw[g][oo][kk] = (o0 + oo < bs && k0 + kk < bs && ZLM_CHK(p, sizeof(TA))) ? to_f32(*p) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < RG_KT; ++kk) {
            const float wr = sw[0][ol][kk], wi = sw[1][ol][kk];
#pragma unroll
            for (int j = 0; j < RG_TT / 4; ++j) {
                const float x = su[tq * (RG_TT / 4) + j][kk];
                acc[0][j] = fmaf(wr, x, acc[0][j]);
                acc[1][j] = fmaf(wi, x, acc[1][j]);
            }
        }
        __syncthreads();
    }
    if (o0 + ol >= bs) return;
    const int c = b * bs + o0 + ol;
    const float br = cr ? to_f32(cr[c]) : 0.f, bi = ci ? to_f32(ci[c]) : 0.f;
#pragma unroll
    for (int j = 0; j < RG_TT / 4; ++j) {
        const int t = t0 + tq * (RG_TT / 4) + j;
        if (t >= T) continue;
        if (ZLM_CHK(zr + (size_t)t * W + c, 4)) zr[(size_t)t * W + c] = acc[0][j] + br;
        if (ZLM_CHK(zi + (size_t)t * W + c, 4)) zi[(size_t)t * W + c] = acc[1][j] + bi;
    }
}

// ---------------------------------------------------------------------------- the recurrence and the y branch
// A thread owns one channel of one sequence: it walks the step's tokens (eight tokens' loads in flight), then leaves the
// state: row 0 the recurrence's S, rows 1 .. taps-1 the newest x + bx.
#define RS_AHEAD 8
template <typename TA>
__global__ void __launch_bounds__(128)
rglru_scan_kernel(TA* __restrict__ out, int out_stride, const float* __restrict__ u, const float* __restrict__ zr,
                  const float* __restrict__ zi, const TA* __restrict__ proj, int proj_stride, int x_off, int y_off,
                  const TA* __restrict__ bx, const TA* __restrict__ by, const TA* __restrict__ lam, float c_decay,
                  float* __restrict__ state, const int* __restrict__ seq_slot, const int* __restrict__ cu_seqlens, int W,
                  int taps, float out_scale) {
    pdl_trigger();
    const int r = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    pdl_wait();
    if (c >= W || !ZLM_CHK(seq_slot + r, 4) || !ZLM_CHK(cu_seqlens + r, 8)) return;
    const int slot = seq_slot[r], row0 = cu_seqlens[r], n = cu_seqlens[r + 1] - row0;
    float* sp = state + (size_t)slot * taps * W + c;
    if (!ZLM_CHK(sp, 4)) return;
    float S = *sp;
    const float sl = softplus_f(to_f32(lam[c])) * c_decay;
    const float yb = by ? to_f32(by[c]) : 0.f;
    for (int s0 = 0; s0 < n; s0 += RS_AHEAD) {
        float vu[RS_AHEAD], vr[RS_AHEAD], vi[RS_AHEAD], vy[RS_AHEAD];
#pragma unroll
        for (int j = 0; j < RS_AHEAD; ++j) {
            const size_t row = (size_t)(row0 + s0 + j);
            const bool ok = s0 + j < n && ZLM_CHK(u + row * W + c, 4) && ZLM_CHK(zr + row * W + c, 4) &&
                            ZLM_CHK(zi + row * W + c, 4) && ZLM_CHK(proj + row * proj_stride + y_off + c, sizeof(TA));
            vu[j] = ok ? u[row * W + c] : 0.f;
            vr[j] = ok ? zr[row * W + c] : 0.f;
            vi[j] = ok ? zi[row * W + c] : 0.f;
            vy[j] = ok ? to_f32(proj[row * proj_stride + y_off + c]) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < RS_AHEAD; ++j) {
            if (s0 + j >= n) break;
            const float log_a = -sigmoid_f(vr[j]) * sl;
            const float a = expf(log_a);
            const float m = sqrtf(fmaxf(-expm1f(2.0f * log_a), 0.f));           // sqrt(1 - a^2) without the cancellation
            S = fmaf(a, S, m * sigmoid_f(vi[j]) * vu[j]);
            TA* dst = out + (size_t)(row0 + s0 + j) * out_stride + c;
            if (ZLM_CHK(dst, sizeof(TA))) *dst = from_f32<TA>(S * gelu_tanh_f(vy[j] + yb) * out_scale);
        }
    }
    *sp = S;
    // the convolution's newest inputs
    const float xb = bx ? to_f32(bx[c]) : 0.f;
    float keep[RC_MAX_TAPS];
    for (int m = 1; m < taps; ++m) {
        const int s = n - taps + m;                  // row m holds the input (taps - m) tokens back from the next one
        if (s >= 0) {
            const TA* p = proj + (size_t)(row0 + s) * proj_stride + x_off + c;
            keep[m] = ZLM_CHK(p, sizeof(TA)) ? to_f32(*p) + xb : 0.f;
        } else {
            keep[m] = sp[(size_t)(taps + s) * W];
        }
    }
    for (int m = 1; m < taps; ++m) sp[(size_t)m * W] = keep[m];
}

template <typename TA>
static void launch_rglru(void* out, int out_stride, float* u, float* zr, float* zi, const void* proj, int proj_stride, int x_off,
                         int y_off, const void* bx, const void* by, const void* conv_w, const void* cb, const void* Ar,
                         const void* Ai, const void* cr, const void* ci, const void* lam, float c_decay, float* state,
                         const int* token_pos, const int* token_slot, const int* token_seq, const int* seq_start,
                         const int* cu_seqlens, const int* seq_slot, int T, int R, int W, int blocks, int taps, float out_scale,
                         cudaStream_t st) {
    const int bs = W / blocks;
    zlm_launch(rglru_conv_kernel<TA>, dim3(T, (W + 255) / 256), dim3(256), 0, st, u, (const TA*)proj, proj_stride, x_off,
               (const TA*)bx, (const TA*)conv_w, (const TA*)cb, (const float*)state, token_pos, token_slot, token_seq, seq_start,
               cu_seqlens, W, taps);
    zlm_launch(rglru_gates_kernel<TA>, dim3((T + RG_TT - 1) / RG_TT, (bs + RG_OT - 1) / RG_OT, blocks), dim3(RG_OT * 4), 0, st, zr,
               zi, (const float*)u, (const TA*)Ar, (const TA*)Ai, (const TA*)cr, (const TA*)ci, T, W, bs);
    zlm_launch(rglru_scan_kernel<TA>, dim3(R, (W + 127) / 128), dim3(128), 0, st, (TA*)out, out_stride, (const float*)u,
               (const float*)zr, (const float*)zi, (const TA*)proj, proj_stride, x_off, y_off, (const TA*)bx, (const TA*)by,
               (const TA*)lam, c_decay, state, seq_slot, cu_seqlens, W, taps, out_scale);
}

// proj [T][proj_stride] holds the x branch from column x_off and the y branch from y_off (W columns each), without their
// biases bx, by [W]; conv_w [W][taps], cb [W]; Ar, Ai [blocks][W/blocks][W/blocks] (out, in), cr, ci [W]; lam [W]; all in
// the element type.  u, zr, zi: fp32 scratch [T][W].  state [slots][taps][W] fp32.  out [T][out_stride] receives
// S * gelu_tanh(y) * out_scale in the element type.
extern "C" int zlm_rglru(void* out, int out_stride, float* u, float* zr, float* zi, const void* proj, int proj_stride, int x_off,
                         int y_off, const void* bx, const void* by, const void* conv_w, const void* cb, const void* Ar,
                         const void* Ai, const void* cr, const void* ci, const void* lam, float c_decay, float* state, int dtype,
                         const int* token_pos, const int* token_slot, const int* token_seq, const int* seq_start,
                         const int* cu_seqlens, const int* seq_slot, int T, int R, int W, int blocks, int taps, float out_scale,
                         cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(W > 0 && blocks > 0 && W % blocks == 0, "rglru: %d channels in %d blocks", W, blocks);
    ZLM_REQUIRE(taps >= 1 && taps <= RC_MAX_TAPS, "rglru: %d taps (at most %d)", taps, RC_MAX_TAPS);
    ZLM_REQUIRE(blocks <= 65535 && (W / blocks + RG_OT - 1) / RG_OT <= 65535 && (W + 127) / 128 <= 65535, "rglru: too many channels");
    if (dtype == ZLM_DTYPE_F32)
        launch_rglru<float>(out, out_stride, u, zr, zi, proj, proj_stride, x_off, y_off, bx, by, conv_w, cb, Ar, Ai, cr, ci, lam,
                            c_decay, state, token_pos, token_slot, token_seq, seq_start, cu_seqlens, seq_slot, T, R, W, blocks,
                            taps, out_scale, st);
    else if (dtype == ZLM_DTYPE_BF16)
        launch_rglru<__nv_bfloat16>(out, out_stride, u, zr, zi, proj, proj_stride, x_off, y_off, bx, by, conv_w, cb, Ar, Ai, cr, ci,
                                    lam, c_decay, state, token_pos, token_slot, token_seq, seq_start, cu_seqlens, seq_slot, T, R,
                                    W, blocks, taps, out_scale, st);
    else
        ZLM_REQUIRE(false, "rglru: unsupported dtype %d", dtype);
    return zlm_check_launch("rglru");
}

// ---------------------------------------------------------------------------- decays from a low-rank projection
// alpha[t][c] = sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau), z = sum_r W2[c][r] lo[t][r] + b[c]; lo: `rank` columns of
// proj from lo_off on.  fp32 throughout.
template <typename TA>
__global__ void __launch_bounds__(256)
lowrank_decay_kernel(float* __restrict__ alpha, const TA* __restrict__ proj, int proj_stride, int lo_off, const TA* __restrict__ W2,
                     const TA* __restrict__ b, int C, int rank, float inv_tau) {
    extern __shared__ float ld_lo[];
    pdl_trigger();
    const int t = blockIdx.x;
    pdl_wait();
    for (int r = threadIdx.x; r < rank; r += blockDim.x) {
        const TA* p = proj + (size_t)t * proj_stride + lo_off + r;
        ld_lo[r] = ZLM_CHK(p, sizeof(TA)) ? to_f32(*p) : 0.f;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float z = b ? to_f32(b[c]) : 0.f;
        for (int r = 0; r < rank; ++r)
            if (ZLM_CHK(W2 + (size_t)c * rank + r, sizeof(TA))) z = fmaf(to_f32(W2[(size_t)c * rank + r]), ld_lo[r], z);
        if (ZLM_CHK(alpha + (size_t)t * C + c, 4)) alpha[(size_t)t * C + c] = expf(-softplus_f(-z) * inv_tau);
    }
}

extern "C" int zlm_lowrank_decay(float* alpha, const void* proj, int proj_stride, int lo_off, const void* W2, const void* b,
                                 int dtype, int T, int C, int rank, float tau, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(C > 0 && rank > 0 && rank <= 8192 && tau > 0.f, "lowrank_decay: %d channels of rank %d, tau %g", C, rank, (double)tau);
    const size_t smem = (size_t)rank * sizeof(float);
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(lowrank_decay_kernel<float>, dim3(T), dim3(256), smem, st, alpha, (const float*)proj, proj_stride, lo_off,
                   (const float*)W2, (const float*)b, C, rank, 1.0f / tau);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(lowrank_decay_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, st, alpha, (const __nv_bfloat16*)proj,
                   proj_stride, lo_off, (const __nv_bfloat16*)W2, (const __nv_bfloat16*)b, C, rank, 1.0f / tau);
    else
        ZLM_REQUIRE(false, "lowrank_decay: unsupported dtype %d", dtype);
    return zlm_check_launch("lowrank_decay");
}

// ---------------------------------------------------------------------------- linear attention with decays per channel
// A block: one head of one sequence and up to 128 value columns; a thread owns one column of the state, DR rows in
// registers (rows from `dim` on stay zero).  The step's tokens are staged LA_CH at a time in shared memory as fp32:
// q (scaled), k, the decays, v.  o [T][H*V] fp32.
#define LA_CH 16
template <typename TA, int DR>
__global__ void __launch_bounds__(128)
linear_attention_kernel(float* __restrict__ o, const TA* __restrict__ proj, int proj_stride, int q_off, int k_off, int v_off,
                        const float* __restrict__ alpha, const float* __restrict__ head_decay, float* __restrict__ state,
                        const int* __restrict__ seq_slot, const int* __restrict__ cu_seqlens, int H, int D, int V,
                        float q_scale) {
    __shared__ __align__(16) float sq[LA_CH][DR], sk[LA_CH][DR], sa[LA_CH][DR];
    __shared__ float sv[LA_CH][128];
    pdl_trigger();
    const int r = blockIdx.x / H, h = blockIdx.x % H, v0 = blockIdx.y * 128, tid = threadIdx.x;
    const int v = v0 + tid;
    pdl_wait();
    if (!ZLM_CHK(seq_slot + r, 4) || !ZLM_CHK(cu_seqlens + r, 8)) return;
    const int slot = seq_slot[r], row0 = cu_seqlens[r], n = cu_seqlens[r + 1] - row0;
    float* sp = state + (((size_t)slot * H + h) * D) * V + v;
    float S[DR];
#pragma unroll
    for (int d = 0; d < DR; ++d) S[d] = (d < D && v < V && ZLM_CHK(sp + (size_t)d * V, 4)) ? sp[(size_t)d * V] : 0.f;
    const float hd = head_decay ? head_decay[h] : 1.0f;
    for (int s0 = 0; s0 < n; s0 += LA_CH) {
        const int m = min(LA_CH, n - s0);
        __syncthreads();
        for (int x = tid; x < LA_CH * DR; x += 128) {
            const int j = x / DR, d = x % DR;
            float fq = 0.f, fk = 0.f, fa = 1.f;
            if (j < m && d < D) {
                const TA* row = proj + (size_t)(row0 + s0 + j) * proj_stride;
                if (ZLM_CHK(row + q_off + h * D + d, sizeof(TA))) fq = to_f32(row[q_off + h * D + d]) * q_scale;
                if (ZLM_CHK(row + k_off + h * D + d, sizeof(TA))) fk = to_f32(row[k_off + h * D + d]);
                if (alpha) {
                    const float* ap = alpha + ((size_t)(row0 + s0 + j) * H + h) * D + d;
                    if (ZLM_CHK(ap, 4)) fa = *ap;
                } else {
                    fa = hd;
                }
            }
            sq[j][d] = fq; sk[j][d] = fk; sa[j][d] = fa;
        }
        for (int x = tid; x < LA_CH * 128; x += 128) {
            const int j = x / 128, e = x % 128;
            float fv = 0.f;
            if (j < m && v0 + e < V) {
                const TA* p = proj + (size_t)(row0 + s0 + j) * proj_stride + v_off + h * V + v0 + e;
                if (ZLM_CHK(p, sizeof(TA))) fv = to_f32(*p);
            }
            sv[j][e] = fv;
        }
        __syncthreads();
        for (int j = 0; j < m; ++j) {
            const float vv = sv[j][tid];
            float acc = 0.f;
#pragma unroll
            for (int d = 0; d < DR; d += 4) {
                const float4 a4 = *(const float4*)&sa[j][d], k4 = *(const float4*)&sk[j][d], q4 = *(const float4*)&sq[j][d];
                S[d] = fmaf(a4.x, S[d], k4.x * vv);         acc = fmaf(S[d], q4.x, acc);
                S[d + 1] = fmaf(a4.y, S[d + 1], k4.y * vv); acc = fmaf(S[d + 1], q4.y, acc);
                S[d + 2] = fmaf(a4.z, S[d + 2], k4.z * vv); acc = fmaf(S[d + 2], q4.z, acc);
                S[d + 3] = fmaf(a4.w, S[d + 3], k4.w * vv); acc = fmaf(S[d + 3], q4.w, acc);
            }
            float* op = o + ((size_t)(row0 + s0 + j) * H + h) * V + v;
            if (v < V && ZLM_CHK(op, 4)) *op = acc;
        }
    }
    if (v < V) {
#pragma unroll
        for (int d = 0; d < DR; ++d)
            if (d < D && ZLM_CHK(sp + (size_t)d * V, 4)) sp[(size_t)d * V] = S[d];
    }
}

// q, k [H*D], v [H*V]: columns of proj from q_off, k_off, v_off on (element type); alpha [T][H*D] fp32 decays per token
// and key channel, or null with head_decay [H] fp32 (one decay a head); state [slots][H][D][V] fp32; o [T][H*V] fp32.
extern "C" int zlm_linear_attention(float* o, const void* proj, int proj_stride, int q_off, int k_off, int v_off,
                                    const float* alpha, const float* head_decay, float* state, int dtype, const int* seq_slot,
                                    const int* cu_seqlens, int T, int R, int H, int D, int V, float q_scale, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(H > 0 && D > 0 && V > 0 && D <= 128, "linear_attention: %d heads of %d key and %d value columns (keys up to 128)", H, D, V);
    ZLM_REQUIRE(alpha || head_decay, "linear_attention: neither decays per channel nor per head");
    ZLM_REQUIRE((long long)R * H <= 2147483647LL && (V + 127) / 128 <= 65535, "linear_attention: too many sequences or columns");
    const dim3 grid(R * H, (V + 127) / 128), block(128);
#define ZLM_LA(TA, DR)                                                                                                     \
    zlm_launch(linear_attention_kernel<TA, DR>, grid, block, 0, st, o, (const TA*)proj, proj_stride, q_off, k_off, v_off, alpha, \
               head_decay, state, seq_slot, cu_seqlens, H, D, V, q_scale)
#define ZLM_LA_D(TA)                                                                     \
    if (D <= 32) ZLM_LA(TA, 32); else if (D <= 64) ZLM_LA(TA, 64); else ZLM_LA(TA, 128)
    if (dtype == ZLM_DTYPE_F32) {
        ZLM_LA_D(float);
    } else if (dtype == ZLM_DTYPE_BF16) {
        ZLM_LA_D(__nv_bfloat16);
    } else {
        ZLM_REQUIRE(false, "linear_attention: unsupported dtype %d", dtype);
    }
#undef ZLM_LA_D
#undef ZLM_LA
    return zlm_check_launch("linear_attention");
}

ZLM_TRANSLATION_UNIT(recurrent)
