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
// steps from the state's rows 1 .. taps-1 (row taps-1 the newest; they hold x + bx), zeros before the start.  u16, if
// given, receives u in the element type as well (the operand of the gates' product on the tensor cores).
template <typename TA>
__global__ void __launch_bounds__(256)
rglru_conv_kernel(float* __restrict__ u, TA* __restrict__ u16, const TA* __restrict__ proj, int proj_stride, int x_off,
                  const TA* __restrict__ bx, const TA* __restrict__ conv_w, const TA* __restrict__ cb,
                  const float* __restrict__ state, const int* __restrict__ token_pos, const int* __restrict__ token_slot,
                  const int* __restrict__ token_seq, const int* __restrict__ seq_start, const int* __restrict__ cu_seqlens,
                  int W, int taps) {
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
    if (u16 && ZLM_CHK(u16 + (size_t)t * W + c, sizeof(TA))) u16[(size_t)t * W + c] = from_f32<TA>(a);
}

// ---------------------------------------------------------------------------- block-diagonal gate logits
// z [T][blocks][2][bs] fp32: z[t][b][g][o] = sum_i A_g[b][o][i] u[t][b*bs + i], g = 0 (recurrence gate), 1 (input gate);
// the gates' biases are added where z is read.  (The same layout as the product u_b [T, bs] x [A_r[b] ; A_i[b]]^T
// leaves, block by block, when the tensor cores compute it.)
// A block: 16 tokens x 64 outputs of one diagonal block, both gates; u and the weights in tiles of 32 inputs in shared
// memory; fp32 multiply-adds in a fixed order.
#define RG_TT 16
#define RG_OT 64
#define RG_KT 32
template <typename TA>
__global__ void __launch_bounds__(RG_OT * 4)
rglru_gates_kernel(float* __restrict__ z, const float* __restrict__ u, const TA* __restrict__ Ar,
                   const TA* __restrict__ Ai, int T, int W, int bs) {
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
#pragma unroll
    for (int j = 0; j < RG_TT / 4; ++j) {
        const int t = t0 + tq * (RG_TT / 4) + j;
        if (t >= T) continue;
        float* zp = z + ((size_t)t * 2 * W) + (size_t)b * 2 * bs + o0 + ol;
        if (ZLM_CHK(zp, 4)) zp[0] = acc[0][j];
        if (ZLM_CHK(zp + bs, 4)) zp[bs] = acc[1][j];
    }
}

// The same for steps of up to 16 tokens: a warp per output channel reads its two rows of the gates' matrices once
// (lanes over the inputs), every token's sums in registers; the lanes' parts meet in a butterfly.
#define RG_FEW 16
// eight neighbouring elements as floats (16 bytes of bf16, 32 of fp32; the caller has checked the alignment)
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
    const uint4 u = *(const uint4*)p;
    f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
    f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
    f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xffff0000u);
    f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xffff0000u);
}
__device__ __forceinline__ void load8(const float* p, float* f) {
    const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// VEC 8: a lane reads eight neighbouring inputs at a time (block sizes that are multiples of 8); VEC 1: one
template <typename TA, int VEC>
__global__ void __launch_bounds__(256)
rglru_gates_few_kernel(float* __restrict__ z, const float* __restrict__ u, const TA* __restrict__ Ar,
                       const TA* __restrict__ Ai, int T, int W, int bs) {
    pdl_trigger();
    const int lane = threadIdx.x & 31, c = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (c >= W) return;
    const int b = c / bs, o = c - b * bs;
    float acc[2][RG_FEW];
#pragma unroll
    for (int t = 0; t < RG_FEW; ++t) acc[0][t] = acc[1][t] = 0.f;
    pdl_wait();
    for (int i = lane * VEC; i < bs; i += 32 * VEC) {
        const TA* pr = Ar + (size_t)c * bs + i;
        const TA* pi = Ai + (size_t)c * bs + i;
        if (!ZLM_CHK(pr, VEC * sizeof(TA)) || !ZLM_CHK(pi, VEC * sizeof(TA))) continue;
        float wr[VEC], wi[VEC];
        if (VEC == 8) { load8(pr, wr); load8(pi, wi); } else { wr[0] = to_f32(*pr); wi[0] = to_f32(*pi); }
#pragma unroll
        for (int t = 0; t < RG_FEW; ++t) {
            if (t >= T) break;
            const float* up = u + (size_t)t * W + b * bs + i;
            if (!ZLM_CHK(up, VEC * 4)) continue;
            float x[VEC];
            if (VEC == 8) load8(up, x); else x[0] = *up;
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                acc[0][t] = fmaf(wr[e], x[e], acc[0][t]);
                acc[1][t] = fmaf(wi[e], x[e], acc[1][t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < RG_FEW; ++t) {
        if (t >= T) break;
        const float sr = warp_sum(acc[0][t]), si = warp_sum(acc[1][t]);
        float* zp = z + ((size_t)t * 2 * W) + (size_t)b * 2 * bs + o;
        if (lane == 0 && ZLM_CHK(zp, 4)) zp[0] = sr;
        if (lane == 0 && ZLM_CHK(zp + bs, 4)) zp[bs] = si;
    }
}

// a token's decay and input: a = exp(-c r softplus(lam)), b = sqrt(1 - a^2) i u, from the gates' logits
__device__ __forceinline__ void rglru_ab(float zr, float zi, float u, float sl, float& a, float& b) {
    const float log_a = -sigmoid_f(zr) * sl;
    a = expf(log_a);
    b = sqrtf(fmaxf(-expm1f(2.0f * log_a), 0.f)) * sigmoid_f(zi) * u;           // sqrt(1 - a^2) without the cancellation
}

// the convolution's newest inputs after a step of n tokens: row m holds the input (taps - m) tokens back from the next
template <typename TA>
__device__ __forceinline__ void rglru_keep_inputs(float* sp, const TA* proj, int proj_stride, int x_off, int c, int row0, int n,
                                                  int W, int taps, float xb) {
    float keep[RC_MAX_TAPS];
    for (int m = 1; m < taps; ++m) {
        const int s = n - taps + m;
        if (s >= 0) {
            const TA* p = proj + (size_t)(row0 + s) * proj_stride + x_off + c;
            keep[m] = ZLM_CHK(p, sizeof(TA)) ? to_f32(*p) + xb : 0.f;
        } else {
            keep[m] = sp[(size_t)(taps + s) * W];
        }
    }
    for (int m = 1; m < taps; ++m) sp[(size_t)m * W] = keep[m];
}

// ---------------------------------------------------------------------------- the recurrence and the y branch
// Short steps: a thread owns one channel of one sequence and walks the step's tokens (eight tokens' loads in flight),
// then leaves the state: row 0 the recurrence's S, rows 1 .. taps-1 the newest x + bx.
#define RS_AHEAD 8
#define PIECE_AHEAD 16          // the pieces' walks: a piece is two such rounds
template <typename TA>
__global__ void __launch_bounds__(128)
rglru_scan_kernel(TA* __restrict__ out, int out_stride, const float* __restrict__ u, const float* __restrict__ z,
                  const TA* __restrict__ proj, int proj_stride, int x_off, int y_off, const TA* __restrict__ bx,
                  const TA* __restrict__ by, const TA* __restrict__ cr, const TA* __restrict__ ci, const TA* __restrict__ lam,
                  float c_decay, float* __restrict__ state, const int* __restrict__ seq_slot,
                  const int* __restrict__ cu_seqlens, int W, int bs, int taps, float out_scale) {
    pdl_trigger();
    const int r = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    pdl_wait();
    if (c >= W || !ZLM_CHK(seq_slot + r, 4) || !ZLM_CHK(cu_seqlens + r, 8)) return;
    const int slot = seq_slot[r], row0 = cu_seqlens[r], n = cu_seqlens[r + 1] - row0;
    float* sp = state + (size_t)slot * taps * W + c;
    if (!ZLM_CHK(sp, 4)) return;
    float S = *sp;
    const float sl = softplus_f(to_f32(lam[c])) * c_decay;
    const float yb = by ? to_f32(by[c]) : 0.f, rb = cr ? to_f32(cr[c]) : 0.f, ib = ci ? to_f32(ci[c]) : 0.f;
    const size_t zc = (size_t)(c / bs) * 2 * bs + (c % bs);
    for (int s0 = 0; s0 < n; s0 += RS_AHEAD) {
        float vu[RS_AHEAD], vr[RS_AHEAD], vi[RS_AHEAD], vy[RS_AHEAD];
#pragma unroll
        for (int j = 0; j < RS_AHEAD; ++j) {
            const size_t row = (size_t)(row0 + s0 + j);
            const bool ok = s0 + j < n && ZLM_CHK(u + row * W + c, 4) && ZLM_CHK(z + row * 2 * W + zc, 4) &&
                            ZLM_CHK(z + row * 2 * W + zc + bs, 4) && ZLM_CHK(proj + row * proj_stride + y_off + c, sizeof(TA));
            vu[j] = ok ? u[row * W + c] : 0.f;
            vr[j] = ok ? z[row * 2 * W + zc] : 0.f;
            vi[j] = ok ? z[row * 2 * W + zc + bs] : 0.f;
            vy[j] = ok ? to_f32(proj[row * proj_stride + y_off + c]) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < RS_AHEAD; ++j) {
            if (s0 + j >= n) break;
            float a, b;
            rglru_ab(vr[j] + rb, vi[j] + ib, vu[j], sl, a, b);
            S = fmaf(a, S, b);
            TA* dst = out + (size_t)(row0 + s0 + j) * out_stride + c;
            if (ZLM_CHK(dst, sizeof(TA))) *dst = from_f32<TA>(S * gelu_tanh_f(vy[j] + yb) * out_scale);
        }
    }
    *sp = S;
    rglru_keep_inputs<TA>(sp, proj, proj_stride, x_off, c, row0, n, W, taps, bx ? to_f32(bx[c]) : 0.f);
}

// Long steps run in pieces of L tokens side by side.  First pass: a thread owns one channel of one piece, turns the
// gates' logits of its tokens into (a, b) in place (a where the recurrence gate's logit stood, b where the input
// gate's stood) and leaves what the piece does to a state: S_out = PA * S_in + PB.
__global__ void __launch_bounds__(128)
rglru_piece_ab_kernel(float* __restrict__ z, const float* __restrict__ u, const void* __restrict__ cr, const void* __restrict__ ci,
                      const void* __restrict__ lam, int dtype, float c_decay, float* __restrict__ PA, float* __restrict__ PB,
                      const int* __restrict__ cu_seqlens, int W, int bs, int maxp, int L) {
    pdl_trigger();
    const int r = blockIdx.x / maxp, p = blockIdx.x % maxp, c = blockIdx.y * blockDim.x + threadIdx.x;
    pdl_wait();
    if (c >= W || !ZLM_CHK(cu_seqlens + r, 8)) return;
    const int row0 = cu_seqlens[r], n = cu_seqlens[r + 1] - row0;
    const int lo = p * L, hi = min(n, lo + L);
    if (lo >= hi) return;
    const VecW vr{cr, dtype}, vi{ci, dtype}, vl{lam, dtype};
    const float sl = softplus_f(vl[c]) * c_decay;
    const float rb = cr ? vr[c] : 0.f, ib = ci ? vi[c] : 0.f;
    const size_t zc = (size_t)(c / bs) * 2 * bs + (c % bs);
    float A = 1.f, B = 0.f;
    for (int s0 = lo; s0 < hi; s0 += PIECE_AHEAD) {
        float fu[PIECE_AHEAD], fr[PIECE_AHEAD], fi[PIECE_AHEAD];
#pragma unroll
        for (int j = 0; j < PIECE_AHEAD; ++j) {
            const size_t row = (size_t)(row0 + s0 + j);
            const bool ok = s0 + j < hi && ZLM_CHK(u + row * W + c, 4) && ZLM_CHK(z + row * 2 * W + zc, 4) && ZLM_CHK(z + row * 2 * W + zc + bs, 4);
            fu[j] = ok ? u[row * W + c] : 0.f;
            fr[j] = ok ? z[row * 2 * W + zc] : 0.f;
            fi[j] = ok ? z[row * 2 * W + zc + bs] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < PIECE_AHEAD; ++j) {
            if (s0 + j >= hi) break;
            float a, b;
            rglru_ab(fr[j] + rb, fi[j] + ib, fu[j], sl, a, b);
            const size_t row = (size_t)(row0 + s0 + j);
            z[row * 2 * W + zc] = a;
            z[row * 2 * W + zc + bs] = b;
            A *= a;
            B = fmaf(a, B, b);
        }
    }
    const size_t at = ((size_t)r * maxp + p) * W + c;
    if (ZLM_CHK(PA + at, 4)) PA[at] = A;
    if (ZLM_CHK(PB + at, 4)) PB[at] = B;
}

// The pieces' states in order: PA[piece] becomes the state the piece starts from; the sequence's state is left.
template <typename TA>
__global__ void __launch_bounds__(128)
rglru_chain_kernel(float* __restrict__ PA, const float* __restrict__ PB, float* __restrict__ state, const TA* __restrict__ proj,
                   int proj_stride, int x_off, const TA* __restrict__ bx, const int* __restrict__ seq_slot,
                   const int* __restrict__ cu_seqlens, int W, int taps, int maxp, int L) {
    pdl_trigger();
    const int r = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    pdl_wait();
    if (c >= W || !ZLM_CHK(seq_slot + r, 4) || !ZLM_CHK(cu_seqlens + r, 8)) return;
    const int slot = seq_slot[r], row0 = cu_seqlens[r], n = cu_seqlens[r + 1] - row0;
    float* sp = state + (size_t)slot * taps * W + c;
    if (!ZLM_CHK(sp, 4)) return;
    float S = *sp;
    const int np = (n + L - 1) / L;
    for (int p0 = 0; p0 < np; p0 += RS_AHEAD) {
        float A[RS_AHEAD], B[RS_AHEAD];
#pragma unroll
        for (int j = 0; j < RS_AHEAD; ++j) {
            const size_t at = ((size_t)r * maxp + p0 + j) * W + c;
            const bool ok = p0 + j < np && ZLM_CHK(PA + at, 4) && ZLM_CHK(PB + at, 4);
            A[j] = ok ? PA[at] : 1.f;
            B[j] = ok ? PB[at] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < RS_AHEAD; ++j) {
            if (p0 + j >= np) break;
            const size_t at = ((size_t)r * maxp + p0 + j) * W + c;
            if (ZLM_CHK(PA + at, 4)) PA[at] = S;
            S = fmaf(A[j], S, B[j]);
        }
    }
    *sp = S;
    rglru_keep_inputs<TA>(sp, proj, proj_stride, x_off, c, row0, n, W, taps, bx ? to_f32(bx[c]) : 0.f);
}

// Second pass: every piece walks its tokens again from the state it starts from.
template <typename TA>
__global__ void __launch_bounds__(128)
rglru_piece_out_kernel(TA* __restrict__ out, int out_stride, const float* __restrict__ z, const float* __restrict__ S0,
                       const TA* __restrict__ proj, int proj_stride, int y_off, const TA* __restrict__ by,
                       const int* __restrict__ cu_seqlens, int W, int bs, int maxp, int L, float out_scale) {
    pdl_trigger();
    const int r = blockIdx.x / maxp, p = blockIdx.x % maxp, c = blockIdx.y * blockDim.x + threadIdx.x;
    pdl_wait();
    if (c >= W || !ZLM_CHK(cu_seqlens + r, 8)) return;
    const int row0 = cu_seqlens[r], n = cu_seqlens[r + 1] - row0;
    const int lo = p * L, hi = min(n, lo + L);
    if (lo >= hi) return;
    const size_t at = ((size_t)r * maxp + p) * W + c;
    float S = ZLM_CHK(S0 + at, 4) ? S0[at] : 0.f;
    const float yb = by ? to_f32(by[c]) : 0.f;
    const size_t zc = (size_t)(c / bs) * 2 * bs + (c % bs);
    for (int s0 = lo; s0 < hi; s0 += PIECE_AHEAD) {
        float fa[PIECE_AHEAD], fb[PIECE_AHEAD], fy[PIECE_AHEAD];
#pragma unroll
        for (int j = 0; j < PIECE_AHEAD; ++j) {
            const size_t row = (size_t)(row0 + s0 + j);
            const bool ok = s0 + j < hi && ZLM_CHK(z + row * 2 * W + zc, 4) && ZLM_CHK(z + row * 2 * W + zc + bs, 4) &&
                            ZLM_CHK(proj + row * proj_stride + y_off + c, sizeof(TA));
            fa[j] = ok ? z[row * 2 * W + zc] : 0.f;
            fb[j] = ok ? z[row * 2 * W + zc + bs] : 0.f;
            fy[j] = ok ? to_f32(proj[row * proj_stride + y_off + c]) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < PIECE_AHEAD; ++j) {
            if (s0 + j >= hi) break;
            S = fmaf(fa[j], S, fb[j]);
            TA* dst = out + (size_t)(row0 + s0 + j) * out_stride + c;
            if (ZLM_CHK(dst, sizeof(TA))) *dst = from_f32<TA>(S * gelu_tanh_f(fy[j] + yb) * out_scale);
        }
    }
}

#define RGLRU_PIECE 32
template <typename TA>
static void launch_rglru(void* out, int out_stride, float* u, void* u16, float* z, int gates_done, const void* proj,
                         int proj_stride, int x_off, int y_off, const void* bx, const void* by, const void* conv_w,
                         const void* cb, const void* Ar, const void* Ai, const void* cr, const void* ci, const void* lam,
                         float c_decay, float* state, const int* token_pos, const int* token_slot, const int* token_seq,
                         const int* seq_start, const int* cu_seqlens, const int* seq_slot, int T, int R, int W, int blocks,
                         int taps, float out_scale, int max_new, float* pieces, int phase, cudaStream_t st) {
    const int bs = W / blocks;
    if (phase == 0 || phase == 1)
        zlm_launch(rglru_conv_kernel<TA>, dim3(T, (W + 255) / 256), dim3(256), 0, st, u, (TA*)u16, (const TA*)proj, proj_stride,
                   x_off, (const TA*)bx, (const TA*)conv_w, (const TA*)cb, (const float*)state, token_pos, token_slot, token_seq,
                   seq_start, cu_seqlens, W, taps);
    if (phase == 1) return;
    if (!gates_done) {
        // (eight inputs a lane where every row of a block starts at a multiple of 16 bytes, and u's rows at 32)
        const bool vec = bs % 8 == 0 && (uintptr_t)Ar % 16 == 0 && (uintptr_t)Ai % 16 == 0 && (uintptr_t)u % 16 == 0;
        if (T <= RG_FEW && vec)
            zlm_launch(rglru_gates_few_kernel<TA, 8>, dim3((W + 7) / 8), dim3(256), 0, st, z, (const float*)u, (const TA*)Ar,
                       (const TA*)Ai, T, W, bs);
        else if (T <= RG_FEW)
            zlm_launch(rglru_gates_few_kernel<TA, 1>, dim3((W + 7) / 8), dim3(256), 0, st, z, (const float*)u, (const TA*)Ar,
                       (const TA*)Ai, T, W, bs);
        else
            zlm_launch(rglru_gates_kernel<TA>, dim3((T + RG_TT - 1) / RG_TT, (bs + RG_OT - 1) / RG_OT, blocks), dim3(RG_OT * 4), 0,
                       st, z, (const float*)u, (const TA*)Ar, (const TA*)Ai, T, W, bs);
    }
    if (pieces) {
        const int L = RGLRU_PIECE, maxp = (max_new + L - 1) / L;
        float* PA = pieces;
        float* PB = pieces + (size_t)R * maxp * W;
        const int dtype = sizeof(TA) == 4 ? ZLM_DTYPE_F32 : ZLM_DTYPE_BF16;
        zlm_launch(rglru_piece_ab_kernel, dim3(R * maxp, (W + 127) / 128), dim3(128), 0, st, z, (const float*)u, cr, ci, lam, dtype,
                   c_decay, PA, PB, cu_seqlens, W, bs, maxp, L);
        zlm_launch(rglru_chain_kernel<TA>, dim3(R, (W + 127) / 128), dim3(128), 0, st, PA, (const float*)PB, state, (const TA*)proj,
                   proj_stride, x_off, (const TA*)bx, seq_slot, cu_seqlens, W, taps, maxp, L);
        zlm_launch(rglru_piece_out_kernel<TA>, dim3(R * maxp, (W + 127) / 128), dim3(128), 0, st, (TA*)out, out_stride,
                   (const float*)z, (const float*)PA, (const TA*)proj, proj_stride, y_off, (const TA*)by, cu_seqlens, W, bs, maxp, L,
                   out_scale);
        return;
    }
    zlm_launch(rglru_scan_kernel<TA>, dim3(R, (W + 127) / 128), dim3(128), 0, st, (TA*)out, out_stride, (const float*)u,
               (const float*)z, (const TA*)proj, proj_stride, x_off, y_off, (const TA*)bx, (const TA*)by, (const TA*)cr,
               (const TA*)ci, (const TA*)lam, c_decay, state, seq_slot, cu_seqlens, W, bs, taps, out_scale);
}

// proj [T][proj_stride] holds the x branch from column x_off and the y branch from y_off (W columns each), without their
// biases bx, by [W]; conv_w [W][taps], cb [W]; Ar, Ai [blocks][W/blocks][W/blocks] (out, in), cr, ci [W]; lam [W]; all in
// the element type.  u: fp32 scratch [T][W]; u16: null, or scratch [T][W] in the element type that receives u as well;
// z: fp32 scratch [T][blocks][2][W/blocks].  state [slots][taps][W] fp32.  out [T][out_stride] receives
// S * gelu_tanh(y) * out_scale in the element type.
// phase 0: everything; 1: the convolution only (the caller then computes z = u16_b [A_r[b] ; A_i[b]]^T block by block
// with a product of its own); 2: what follows the gates' logits (gates_done 1: z holds them).
// pieces: null (a thread walks a sequence's tokens), or 2 * R * ceil(max_new / 32) * W floats: sequences run in pieces of
// 32 tokens side by side.
extern "C" int zlm_rglru(void* out, int out_stride, float* u, void* u16, float* z, const void* proj, int proj_stride, int x_off,
                         int y_off, const void* bx, const void* by, const void* conv_w, const void* cb, const void* Ar,
                         const void* Ai, const void* cr, const void* ci, const void* lam, float c_decay, float* state, int dtype,
                         const int* token_pos, const int* token_slot, const int* token_seq, const int* seq_start,
                         const int* cu_seqlens, const int* seq_slot, int T, int R, int W, int blocks, int taps, float out_scale,
                         int max_new, float* pieces, int phase, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(W > 0 && blocks > 0 && W % blocks == 0, "rglru: %d channels in %d blocks", W, blocks);
    ZLM_REQUIRE(taps >= 1 && taps <= RC_MAX_TAPS, "rglru: %d taps (at most %d)", taps, RC_MAX_TAPS);
    ZLM_REQUIRE(blocks <= 65535 && (W / blocks + RG_OT - 1) / RG_OT <= 65535 && (W + 127) / 128 <= 65535, "rglru: too many channels");
    ZLM_REQUIRE(phase >= 0 && phase <= 2 && (!pieces || max_new > 0), "rglru: phase %d, longest sequence %d", phase, max_new);
    const int gates_done = phase == 2 ? 1 : 0;
    if (dtype == ZLM_DTYPE_F32)
        launch_rglru<float>(out, out_stride, u, u16, z, gates_done, proj, proj_stride, x_off, y_off, bx, by, conv_w, cb, Ar, Ai, cr,
                            ci, lam, c_decay, state, token_pos, token_slot, token_seq, seq_start, cu_seqlens, seq_slot, T, R, W,
                            blocks, taps, out_scale, max_new, pieces, phase, st);
    else if (dtype == ZLM_DTYPE_BF16)
        launch_rglru<__nv_bfloat16>(out, out_stride, u, u16, z, gates_done, proj, proj_stride, x_off, y_off, bx, by, conv_w, cb, Ar,
                                    Ai, cr, ci, lam, c_decay, state, token_pos, token_slot, token_seq, seq_start, cu_seqlens,
                                    seq_slot, T, R, W, blocks, taps, out_scale, max_new, pieces, phase, st);
    else
        ZLM_REQUIRE(false, "rglru: unsupported dtype %d", dtype);
    return zlm_check_launch("rglru");
}

// ---------------------------------------------------------------------------- decays from a low-rank projection
// alpha[t][c] = sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau), z = sum_r W2[c][r] lo[t][r] + b[c]; lo: `rank` columns of
// proj from lo_off on.  fp32 throughout.
// TOK tokens a block: a thread reads its channel's row of W2 once for all of them
template <typename TA, int TOK>
__global__ void __launch_bounds__(256)
lowrank_decay_kernel(float* __restrict__ alpha, const TA* __restrict__ proj, int proj_stride, int lo_off, const TA* __restrict__ W2,
                     const TA* __restrict__ b, int T, int C, int rank, float inv_tau) {
    extern __shared__ float ld_lo[];            // [TOK][rank]
    pdl_trigger();
    const int t0 = blockIdx.x * TOK;
    pdl_wait();
    for (int x = threadIdx.x; x < TOK * rank; x += blockDim.x) {
        const int tt = x / rank, r = x - tt * rank;
        const TA* p = proj + (size_t)(t0 + tt) * proj_stride + lo_off + r;
        ld_lo[x] = (t0 + tt < T && ZLM_CHK(p, sizeof(TA))) ? to_f32(*p) : 0.f;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float z[TOK];
        const float bias = b ? to_f32(b[c]) : 0.f;
#pragma unroll
        for (int tt = 0; tt < TOK; ++tt) z[tt] = bias;
        for (int r = 0; r < rank; ++r) {
            if (!ZLM_CHK(W2 + (size_t)c * rank + r, sizeof(TA))) continue;
            const float w = to_f32(W2[(size_t)c * rank + r]);
#pragma unroll
            for (int tt = 0; tt < TOK; ++tt) z[tt] = fmaf(w, ld_lo[tt * rank + r], z[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < TOK; ++tt) {
            if (t0 + tt >= T) break;
            float* ap = alpha + (size_t)(t0 + tt) * C + c;
            if (ZLM_CHK(ap, 4)) *ap = expf(-softplus_f(-z[tt]) * inv_tau);
        }
    }
}

extern "C" int zlm_lowrank_decay(float* alpha, const void* proj, int proj_stride, int lo_off, const void* W2, const void* b,
                                 int dtype, int T, int C, int rank, float tau, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(C > 0 && rank > 0 && rank <= 512 && tau > 0.f, "lowrank_decay: %d channels of rank %d, tau %g", C, rank, (double)tau);
    // many tokens: sixteen a block; few: one, so that the blocks are many
#define ZLM_LD(TA, TOK)                                                                                                  \
    zlm_launch(lowrank_decay_kernel<TA, TOK>, dim3((T + TOK - 1) / TOK), dim3(256), (size_t)TOK * rank * sizeof(float), st, alpha, \
               (const TA*)proj, proj_stride, lo_off, (const TA*)W2, (const TA*)b, T, C, rank, 1.0f / tau)
    if (dtype == ZLM_DTYPE_F32) {
        if (T >= 256) ZLM_LD(float, 16); else ZLM_LD(float, 1);
    } else if (dtype == ZLM_DTYPE_BF16) {
        if (T >= 256) ZLM_LD(__nv_bfloat16, 16); else ZLM_LD(__nv_bfloat16, 1);
    } else {
        ZLM_REQUIRE(false, "lowrank_decay: unsupported dtype %d", dtype);
    }
#undef ZLM_LD
    return zlm_check_launch("lowrank_decay");
}

// ---------------------------------------------------------------------------- linear attention with decays per channel
// A block: one head of one sequence (or of one piece of a sequence) and up to 128 value columns; a thread owns one
// column of the state, DR rows in registers (rows from `dim` on stay zero).  The tokens are staged LA_CH at a time in
// shared memory as fp32: q (scaled), k, the decays, v.  o [T][H*V] fp32.
//   MODE 0: a sequence's tokens in order, from and to the sequence's state.
//   MODE 1: a piece of L tokens from a zero state; leaves the piece's outputs, the state it ends with (part) and the
//           product of its decays per key channel (pdecay): S_out = diag(pdecay) S_in + part.
//   MODE 2: the piece again from the state it really starts with (part, after the chain), without keys and values:
//           o_t += (diag(alpha_lo .. alpha_t) S_in)^T q_t.
#define LA_CH 16
template <typename TA, int DR, int MODE>
__global__ void __launch_bounds__(128)
linear_attention_kernel(float* __restrict__ o, const TA* __restrict__ proj, int proj_stride, int q_off, int k_off, int v_off,
                        const float* __restrict__ alpha, const float* __restrict__ head_decay, float* __restrict__ state,
                        const int* __restrict__ seq_slot, const int* __restrict__ cu_seqlens, int H, int D, int V,
                        float q_scale, float* __restrict__ part, float* __restrict__ pdecay, int maxp, int L) {
    __shared__ __align__(16) float sq[LA_CH][DR], sk[LA_CH][DR], sa[LA_CH][DR];
    __shared__ float sv[LA_CH][128];
    pdl_trigger();
    const int unit = blockIdx.x / H, h = blockIdx.x % H, v0 = blockIdx.y * 128, tid = threadIdx.x;
    const int r = MODE == 0 ? unit : unit / maxp, p = MODE == 0 ? 0 : unit % maxp;
    const int v = v0 + tid;
    pdl_wait();
    if (!ZLM_CHK(seq_slot + r, 4) || !ZLM_CHK(cu_seqlens + r, 8)) return;
    const int slot = seq_slot[r], row0 = cu_seqlens[r], n = cu_seqlens[r + 1] - row0;
    const int lo = MODE == 0 ? 0 : p * L, hi = MODE == 0 ? n : min(n, lo + L);
    if (lo >= hi) return;
    float* sp = MODE == 0 ? state + (((size_t)slot * H + h) * D) * V + v
                          : part + ((((size_t)r * maxp + p) * H + h) * D) * V + v;
    float S[DR];
#pragma unroll
    for (int d = 0; d < DR; ++d)
        S[d] = (MODE != 1 && d < D && v < V && ZLM_CHK(sp + (size_t)d * V, 4)) ? sp[(size_t)d * V] : 0.f;
    const float hd = head_decay ? head_decay[h] : 1.0f;
    float pd = 1.0f;                              // MODE 1: the product of the piece's decays of key channel `tid`
    for (int s0 = lo; s0 < hi; s0 += LA_CH) {
        const int m = min(LA_CH, hi - s0);
        __syncthreads();
        for (int x = tid; x < LA_CH * DR; x += 128) {
            const int j = x / DR, d = x % DR;
            float fq = 0.f, fk = 0.f, fa = 1.f;
            if (j < m && d < D) {
                const TA* row = proj + (size_t)(row0 + s0 + j) * proj_stride;
                if (ZLM_CHK(row + q_off + h * D + d, sizeof(TA))) fq = to_f32(row[q_off + h * D + d]) * q_scale;
                if (MODE != 2 && ZLM_CHK(row + k_off + h * D + d, sizeof(TA))) fk = to_f32(row[k_off + h * D + d]);
                if (alpha) {
                    const float* ap = alpha + ((size_t)(row0 + s0 + j) * H + h) * D + d;
                    if (ZLM_CHK(ap, 4)) fa = *ap;
                } else {
                    fa = hd;
                }
            }
            sq[j][d] = fq; sk[j][d] = fk; sa[j][d] = fa;
        }
        if (MODE != 2) {
            for (int x = tid; x < LA_CH * 128; x += 128) {
                const int j = x / 128, e = x % 128;
                float fv = 0.f;
                if (j < m && v0 + e < V) {
                    const TA* pv = proj + (size_t)(row0 + s0 + j) * proj_stride + v_off + h * V + v0 + e;
                    if (ZLM_CHK(pv, sizeof(TA))) fv = to_f32(*pv);
                }
                sv[j][e] = fv;
            }
        }
        __syncthreads();
        if (MODE == 1 && tid < DR)
            for (int j = 0; j < m; ++j) pd *= sa[j][tid];
        for (int j = 0; j < m; ++j) {
            const float vv = MODE == 2 ? 0.f : sv[j][tid];
            float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;         // four sums side by side (always added in this order)
#pragma unroll
            for (int d = 0; d < DR; d += 4) {
                const float4 a4 = *(const float4*)&sa[j][d], q4 = *(const float4*)&sq[j][d];
                if (MODE == 2) {
                    S[d] *= a4.x;     c0 = fmaf(S[d], q4.x, c0);
                    S[d + 1] *= a4.y; c1 = fmaf(S[d + 1], q4.y, c1);
                    S[d + 2] *= a4.z; c2 = fmaf(S[d + 2], q4.z, c2);
                    S[d + 3] *= a4.w; c3 = fmaf(S[d + 3], q4.w, c3);
                } else {
                    const float4 k4 = *(const float4*)&sk[j][d];
                    S[d] = fmaf(a4.x, S[d], k4.x * vv);         c0 = fmaf(S[d], q4.x, c0);
                    S[d + 1] = fmaf(a4.y, S[d + 1], k4.y * vv); c1 = fmaf(S[d + 1], q4.y, c1);
                    S[d + 2] = fmaf(a4.z, S[d + 2], k4.z * vv); c2 = fmaf(S[d + 2], q4.z, c2);
                    S[d + 3] = fmaf(a4.w, S[d + 3], k4.w * vv); c3 = fmaf(S[d + 3], q4.w, c3);
                }
            }
            const float acc = (c0 + c1) + (c2 + c3);
            float* op = o + ((size_t)(row0 + s0 + j) * H + h) * V + v;
            if (v < V && ZLM_CHK(op, 4)) *op = MODE == 2 ? *op + acc : acc;
        }
    }
    if (MODE != 2 && v < V) {
#pragma unroll
        for (int d = 0; d < DR; ++d)
            if (d < D && ZLM_CHK(sp + (size_t)d * V, 4)) sp[(size_t)d * V] = S[d];
    }
    if (MODE == 1 && blockIdx.y == 0 && tid < D) {
        float* pp = pdecay + (((size_t)r * maxp + p) * H + h) * D + tid;
        if (ZLM_CHK(pp, 4)) *pp = pd;
    }
}

// The pieces' states in order: part[piece] becomes the state the piece starts from, the sequence's state is left.
// (a thread owns one number of the state; eight pieces' loads in flight)
#define CHAIN_AHEAD 8
__global__ void __launch_bounds__(128)
linear_attention_chain_kernel(float* __restrict__ part, const float* __restrict__ pdecay, float* __restrict__ state,
                              const int* __restrict__ seq_slot, const int* __restrict__ cu_seqlens, int H, int D, int V,
                              int maxp, int L) {
    pdl_trigger();
    const int d = blockIdx.x % D, rh = blockIdx.x / D, r = rh / H, h = rh % H, v = blockIdx.y * 128 + threadIdx.x;
    pdl_wait();
    if (v >= V || !ZLM_CHK(seq_slot + r, 4) || !ZLM_CHK(cu_seqlens + r, 8)) return;
    const int slot = seq_slot[r], n = cu_seqlens[r + 1] - cu_seqlens[r];
    const int np = (n + L - 1) / L;
    float* sp = state + (((size_t)slot * H + h) * D + d) * V + v;
    if (!ZLM_CHK(sp, 4)) return;
    float S = *sp;
    const size_t pstride = (size_t)H * D * V, dstride = (size_t)H * D;
    float* pp = part + (((size_t)r * maxp * H + h) * D + d) * V + v;
    const float* dp = pdecay + ((size_t)r * maxp * H + h) * D + d;
    for (int p0 = 0; p0 < np; p0 += CHAIN_AHEAD) {
        float A[CHAIN_AHEAD], g[CHAIN_AHEAD];
#pragma unroll
        for (int j = 0; j < CHAIN_AHEAD; ++j) {
            const bool ok = p0 + j < np && ZLM_CHK(pp + (p0 + j) * pstride, 4) && ZLM_CHK(dp + (p0 + j) * dstride, 4);
            A[j] = ok ? pp[(p0 + j) * pstride] : 0.f;
            g[j] = ok ? dp[(p0 + j) * dstride] : 1.f;
        }
#pragma unroll
        for (int j = 0; j < CHAIN_AHEAD; ++j) {
            if (p0 + j >= np) break;
            if (ZLM_CHK(pp + (p0 + j) * pstride, 4)) pp[(p0 + j) * pstride] = S;
            S = fmaf(g[j], S, A[j]);
        }
    }
    *sp = S;
}

#define LA_PIECE 32
// q, k [H*D], v [H*V]: columns of proj from q_off, k_off, v_off on (element type); alpha [T][H*D] fp32 decays per token
// and key channel, or null with head_decay [H] fp32 (one decay a head); state [slots][H][D][V] fp32; o [T][H*V] fp32.
// pieces: null, or R * ceil(max_new / 64) * H * D * (V + 1) floats: sequences run in pieces of 32 tokens side by side
// (two passes and a chain between them).
extern "C" int zlm_linear_attention(float* o, const void* proj, int proj_stride, int q_off, int k_off, int v_off,
                                    const float* alpha, const float* head_decay, float* state, int dtype, const int* seq_slot,
                                    const int* cu_seqlens, int T, int R, int H, int D, int V, float q_scale, int max_new,
                                    float* pieces, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(H > 0 && D > 0 && V > 0 && D <= 128, "linear_attention: %d heads of %d key and %d value columns (keys up to 128)", H, D, V);
    ZLM_REQUIRE(alpha || head_decay, "linear_attention: neither decays per channel nor per head");
    ZLM_REQUIRE(!pieces || max_new > 0, "linear_attention: pieces without the longest sequence");
    const int L = LA_PIECE, maxp = pieces ? (max_new + L - 1) / L : 1;
    ZLM_REQUIRE((long long)R * H * maxp <= 2147483647LL && (long long)R * H * D <= 2147483647LL && (V + 127) / 128 <= 65535, "linear_attention: too many sequences or columns");
    const dim3 grid(R * H, (V + 127) / 128), pgrid(R * maxp * H, (V + 127) / 128), block(128);
    float* part = pieces;
    float* pdecay = pieces ? pieces + (size_t)R * maxp * H * D * V : nullptr;
#define ZLM_LA(TA, DR, MODE, G)                                                                                                \
    zlm_launch(linear_attention_kernel<TA, DR, MODE>, G, block, 0, st, o, (const TA*)proj, proj_stride, q_off, k_off, v_off, alpha, \
               head_decay, state, seq_slot, cu_seqlens, H, D, V, q_scale, part, pdecay, maxp, L)
#define ZLM_LA_RUN(TA, DR)                                                                                                 \
    do {                                                                                                                   \
        if (!pieces) { ZLM_LA(TA, DR, 0, grid); break; }                                                                   \
        ZLM_LA(TA, DR, 1, pgrid);                                                                                          \
        zlm_launch(linear_attention_chain_kernel, dim3(R * H * D, (V + 127) / 128), block, 0, st, part,                \
                   (const float*)pdecay, state, seq_slot, cu_seqlens, H, D, V, maxp, L);                                                                          \
        ZLM_LA(TA, DR, 2, pgrid);                                                                                          \
    } while (0)
#define ZLM_LA_D(TA)                                                                     \
    if (D <= 32) ZLM_LA_RUN(TA, 32); else if (D <= 64) ZLM_LA_RUN(TA, 64); else ZLM_LA_RUN(TA, 128)
    if (dtype == ZLM_DTYPE_F32) {
        ZLM_LA_D(float);
    } else if (dtype == ZLM_DTYPE_BF16) {
        ZLM_LA_D(__nv_bfloat16);
    } else {
        ZLM_REQUIRE(false, "linear_attention: unsupported dtype %d", dtype);
    }
#undef ZLM_LA_D
#undef ZLM_LA_RUN
#undef ZLM_LA
    return zlm_check_launch("linear_attention");
}

ZLM_TRANSLATION_UNIT(recurrent)
