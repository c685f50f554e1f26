// Routed feed-forward (mixture of experts), the plain kernels for both element types and every size:
//   moe_route     per token: router logits z = W_r h in fp32, scores sigmoid(z) (or softmax), the `top`
//                 largest (ties to the lower index) with their scores as weights; optionally a gate
//                 sigmoid(w_g . h) for a shared expert
//   moe_up        a[t, j, f] = act(w_tj * (W_up[e_tj] h_t)[f]): the weight scales the expert's input, which
//                 for a bias-free expert is the same as scaling its first product
//   moe_down      stream[t, :] += sum_j W_down[e_tj] a[t, j, :], experts in the order they were chosen
//   act_scale     out[t, i] = act(u[t, i]) * s[t]  (a shared expert between the library's dense products)
// act is relu(z)^2.  A warp owns one output and shares the inner dimension among its lanes, so every sum's
// order depends on the sizes alone, not on the batch.
#include "common.cuh"

// eight consecutive elements from 16-byte aligned storage as floats
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
    const uint4 v = *(const uint4*)p;
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ void load8(const float* p, float* f) {
    const float4 a = *(const float4*)p, b = *(const float4*)(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// sum_k w[k] x[k] by one warp; `vec`: K % 8 == 0 and both rows 16-byte aligned
template <typename TA>
__device__ __forceinline__ float warp_dot(const TA* __restrict__ w, const TA* __restrict__ x, int K, int lane, bool vec) {
    float acc = 0.f;
    if (vec) {
        for (int k = lane * 8; k < K; k += 256) {
            if (!ZLM_CHK(w + k, 8 * sizeof(TA)) || !ZLM_CHK(x + k, 8 * sizeof(TA))) continue;
            float a[8], b[8];
            load8(w + k, a);
            load8(x + k, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc = fmaf(a[i], b[i], acc);
        }
    } else {
        for (int k = lane; k < K; k += 32)
            if (ZLM_CHK(w + k, sizeof(TA)) && ZLM_CHK(x + k, sizeof(TA))) acc = fmaf(to_f32(w[k]), to_f32(x[k]), acc);
    }
    return warp_sum(acc);
}

template <typename TA>
__device__ __forceinline__ bool rows_vectorise(const TA* a, const TA* b, int K, size_t lda, size_t ldb) {
    return K % 8 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)b % 16 == 0 && (lda * sizeof(TA)) % 16 == 0 &&
           (ldb * sizeof(TA)) % 16 == 0;
}

// ---------------------------------------------------------------------------- router
// One warp chooses for one token.  sc[E] holds the logits (score_kind 1) or the scores (0) and is left holding the
// scores; cs[E] and gm[groups] are scratch.  The choice is made by the scores plus `corr` (if given); the experts
// form `groups` equal groups of neighbours of which only the `keep` with the largest best choice score can be
// chosen; ties go to the lower index.  The weights are the chosen experts' scores (without corr) times wscale,
// divided by their sum first if renorm.
__device__ __forceinline__ void warp_argmax(const float* v, int n, int lane, float& bv, int& bi) {
    bv = -INFINITY;
    bi = 0x7fffffff;
    for (int e = lane; e < n; e += 32) {
        const float x = v[e];
        if (x > bv) { bv = x; bi = e; }            // ascending e: ties keep the lower index
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
}

__device__ __forceinline__ void route_choose(float* sc, float* cs, float* gm, int* __restrict__ idx, float* __restrict__ wgt,
                                             int t, int lane, int E, int top, int score_kind, int renorm,
                                             const float* __restrict__ corr, int groups, int keep, int group_top, float wscale) {
    if (score_kind == 1) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, sc[e]);
        mx = warp_max(mx);
        // every lane adds its share, then the lanes' sums meet in a butterfly: the same bits in every lane, in an
        // order that depends on E alone
        float part = 0.f;
        for (int e = lane; e < E; e += 32) part += expf(sc[e] - mx);
        const float sum = warp_sum(part);
        __syncwarp();
        for (int e = lane; e < E; e += 32) sc[e] = expf(sc[e] - mx) / sum;
        __syncwarp();
    }
    for (int e = lane; e < E; e += 32) cs[e] = sc[e] + ((corr && ZLM_CHK(corr + e, 4)) ? corr[e] : 0.f);
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int size = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float m = -INFINITY, m2 = -INFINITY;                    // the group's largest and second largest choice score
            for (int e = g * size; e < (g + 1) * size; ++e) {
                const float x = cs[e];
                if (x > m) { m2 = m; m = x; } else if (x > m2) { m2 = x; }
            }
            gm[g] = (group_top >= 2 && size >= 2) ? m + m2 : m;
        }
        __syncwarp();
        for (int j = 0; j < keep; ++j) {
            float bv;
            int bi;
            warp_argmax(gm, groups, lane, bv, bi);
            if (lane == 0 && bi < groups) gm[bi] = -INFINITY;       // kept (choice scores are finite)
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gm[e / size] != -INFINITY) cs[e] = -INFINITY;       // not among the best groups
        __syncwarp();
    }
    float chosen_sum = 0.f;
    for (int j = 0; j < top; ++j) {
        float bv;
        int bi;
        warp_argmax(cs, E, lane, bv, bi);
        if (bi >= E) bi = 0;                                        // (fewer candidates than top: refused by the host)
        const float s = sc[bi];
        if (lane == 0 && ZLM_CHK(idx + (size_t)t * top + j, 4) && ZLM_CHK(wgt + (size_t)t * top + j, 4)) {
            idx[(size_t)t * top + j] = bi;
            wgt[(size_t)t * top + j] = s * wscale;
            cs[bi] = -INFINITY;
        }
        chosen_sum += s;
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int j = 0; j < top; ++j) wgt[(size_t)t * top + j] /= chosen_sum;
}

#define ROUTE_WARPS 32
// TOK tokens a block: a warp computes one expert's logit for all of them from one pass over the expert's row
// (steps of many tokens would otherwise read the router's matrix once per token from L2); then warp j chooses
// for token j.  score_kind 0: sigmoid of each logit; 1: softmax over the experts.  renorm: the chosen weights
// divided by their sum.
template <typename TA, int TOK>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(int* __restrict__ idx, float* __restrict__ wgt, float* __restrict__ gate, const TA* __restrict__ x,
                 int x_stride, const TA* __restrict__ Wr, const TA* __restrict__ wg, int T, int E, int K, int top,
                 int score_kind, int renorm, const float* __restrict__ corr, int groups, int keep, int group_top, float wscale) {
    extern __shared__ float sc_all[];           // [TOK][2E + groups]: scores, choice scores, the groups' best
    pdl_trigger();
    const int t0 = blockIdx.x * TOK, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    const bool vec = rows_vectorise(Wr, x, K, (size_t)K, (size_t)x_stride) && (wg == nullptr || (uintptr_t)wg % 16 == 0);
    for (int e = warp; e < E + (wg ? 1 : 0); e += ROUTE_WARPS) {
        const TA* w = e < E ? Wr + (size_t)e * K : wg;
        float acc[TOK];
#pragma unroll
        for (int j = 0; j < TOK; ++j) acc[j] = 0.f;
        if (vec) {
            for (int k = lane * 8; k < K; k += 256) {
                if (!ZLM_CHK(w + k, 8 * sizeof(TA))) continue;
                float a[8], b[8];
                load8(w + k, a);
#pragma unroll
                for (int j = 0; j < TOK; ++j) {
                    const TA* xr = x + (size_t)min(t0 + j, T - 1) * x_stride;
                    if (!ZLM_CHK(xr + k, 8 * sizeof(TA))) continue;
                    load8(xr + k, b);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[j] = fmaf(a[i], b[i], acc[j]);
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) {
                if (!ZLM_CHK(w + k, sizeof(TA))) continue;
                const float a = to_f32(w[k]);
#pragma unroll
                for (int j = 0; j < TOK; ++j) {
                    const TA* xr = x + (size_t)min(t0 + j, T - 1) * x_stride;
                    if (ZLM_CHK(xr + k, sizeof(TA))) acc[j] = fmaf(a, to_f32(xr[k]), acc[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < TOK; ++j) {
            const float z = warp_sum(acc[j]);
            if (lane == 0 && t0 + j < T) {
                if (e < E) sc_all[j * (2 * E + groups) + e] = score_kind == 0 ? 1.0f / (1.0f + expf(-z)) : z;
                else if (ZLM_CHK(gate + t0 + j, 4)) gate[t0 + j] = 1.0f / (1.0f + expf(-z));
            }
        }
    }
    __syncthreads();
    if (warp >= TOK || t0 + warp >= T) return;
    float* sc = sc_all + warp * (2 * E + groups);
    route_choose(sc, sc + E, sc + 2 * E, idx, wgt, t0 + warp, lane, E, top, score_kind, renorm, corr, groups, keep, group_top, wscale);
}

// The same choice from logits that a product of the library left in fp32 (bf16 steps: the router's matrix, with the
// shared expert's gate as one more row, goes through the tensor cores like any other product with fp32 sums):
// logits [T, ld] with E expert columns and, if has_gate, the gate's logit in column E.  One warp per token.
__global__ void __launch_bounds__(128)
moe_choose_kernel(int* __restrict__ idx, float* __restrict__ wgt, float* __restrict__ gate, const float* __restrict__ logits,
                  int ld, int T, int E, int top, int has_gate, int score_kind, int renorm, const float* __restrict__ corr,
                  int groups, int keep, int group_top, float wscale) {
    extern __shared__ float sc_all[];           // [4][2E + groups]
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 4 + warp;
    pdl_wait();
    if (t >= T) return;
    float* sc = sc_all + warp * (2 * E + groups);
    const float* z = logits + (size_t)t * ld;
    for (int e = lane; e < E; e += 32)
        if (ZLM_CHK(z + e, 4)) sc[e] = score_kind == 0 ? 1.0f / (1.0f + expf(-z[e])) : z[e];
    if (has_gate && lane == 0 && ZLM_CHK(z + E, 4) && ZLM_CHK(gate + t, 4)) gate[t] = 1.0f / (1.0f + expf(-z[E]));
    __syncwarp();
    route_choose(sc, sc + E, sc + 2 * E, idx, wgt, t, lane, E, top, score_kind, renorm, corr, groups, keep, group_top, wscale);
}

static int route_groups_ok(int E, int top, int groups, int keep) {
    ZLM_REQUIRE(groups >= 1 && keep >= 1 && keep <= groups && E % groups == 0 && (long long)keep * (E / groups) >= top,
                "moe routing: %d groups of %d experts of which %d are kept cannot give %d choices", groups, E / (groups > 0 ? groups : 1), keep, top);
    return ZLM_OK;
}

// corr (fp32 [E], may be null): added to the scores for the choice only; groups / keep: the experts form `groups` equal
// groups of neighbours and only the `keep` best groups (by their largest choice score) can be chosen; wscale multiplies
// the weights.  1, 1, 1.0 and no corr give the plain top-k.
extern "C" int zlm_moe_choose(int* idx, float* wgt, float* gate, const float* logits, int ld, int T, int E, int top,
                              int has_gate, int score_kind, int renorm, const float* corr, int groups, int keep, int group_top,
                              float wscale, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    if (int rc = route_groups_ok(E, top, groups, keep)) return rc;
    ZLM_REQUIRE(E > 0 && E <= 2048 && top > 0 && top <= E && ld >= E + (has_gate ? 1 : 0), "moe_choose: experts=%d top=%d ld=%d", E, top, ld);
    ZLM_REQUIRE(!has_gate || gate, "moe_choose: a shared gate needs a place for its values");
    zlm_launch(moe_choose_kernel, (T + 3) / 4, 128, (size_t)4 * (2 * E + groups) * sizeof(float), st, idx, wgt, gate, logits, ld,
               T, E, top, has_gate, score_kind, renorm, corr, groups, keep, group_top, wscale);
    return zlm_check_launch("moe_choose");
}

template <typename TA>
static void launch_route(int* idx, float* wgt, float* gate, const void* x, int x_stride, const void* Wr, const void* wg,
                         int T, int E, int K, int top, int score_kind, int renorm, const float* corr, int groups, int keep, int group_top,
                         float wscale, cudaStream_t st) {
    // many tokens: four a block (a quarter of the reads of the router's matrix); few: one, so that the blocks are many
    if (T >= 64)
        zlm_launch(moe_route_kernel<TA, 4>, (T + 3) / 4, ROUTE_WARPS * 32, (size_t)4 * (2 * E + groups) * sizeof(float), st, idx,
                   wgt, gate, (const TA*)x, x_stride, (const TA*)Wr, (const TA*)wg, T, E, K, top, score_kind, renorm, corr, groups,
                   keep, group_top, wscale);
    else
        zlm_launch(moe_route_kernel<TA, 1>, T, ROUTE_WARPS * 32, (size_t)(2 * E + groups) * sizeof(float), st, idx, wgt, gate,
                   (const TA*)x, x_stride, (const TA*)Wr, (const TA*)wg, T, E, K, top, score_kind, renorm, corr, groups, keep, group_top,
                   wscale);
}

extern "C" int zlm_moe_route(int* idx, float* wgt, float* gate, const void* x, int x_stride, const void* Wr,
                             const void* wg, int dtype, int T, int E, int K, int top, int score_kind, int renorm,
                             const float* corr, int groups, int keep, int group_top, float wscale, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    if (int rc = route_groups_ok(E, top, groups, keep)) return rc;
    ZLM_REQUIRE(E > 0 && E <= 2048 && K > 0 && top > 0 && top <= E, "moe_route: experts=%d top=%d K=%d", E, top, K);
    ZLM_REQUIRE(score_kind == 0 || score_kind == 1, "moe_route: score kind %d", score_kind);
    ZLM_REQUIRE(wg == nullptr || gate != nullptr, "moe_route: a shared gate needs a place for its values");
    if (dtype == ZLM_DTYPE_F32)
        launch_route<float>(idx, wgt, gate, x, x_stride, Wr, wg, T, E, K, top, score_kind, renorm, corr, groups, keep, group_top, wscale, st);
    else if (dtype == ZLM_DTYPE_BF16)
        launch_route<__nv_bfloat16>(idx, wgt, gate, x, x_stride, Wr, wg, T, E, K, top, score_kind, renorm, corr, groups, keep, group_top,
                                    wscale, st);
    else
        ZLM_REQUIRE(false, "moe_route: unsupported dtype %d", dtype);
    return zlm_check_launch("moe_route");
}

// ---------------------------------------------------------------------------- experts, token by token
__device__ __forceinline__ float relu2(float z) { z = fmaxf(z, 0.f); return z * z; }

#define MOE_WARPS 8
// act[t, j, f] = relu(w[t, j] * (Wup[idx[t, j]][f, :] . x[t]))^2;  grid (ceil(F / MOE_WARPS), top, T)
template <typename TA>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_up_kernel(TA* __restrict__ act, const TA* __restrict__ x, int x_stride, const TA* __restrict__ Wup,
              const int* __restrict__ idx, const float* __restrict__ wgt, int top, int F, int K, int scale_input, int act_kind,
              int n_real) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int f = blockIdx.x * MOE_WARPS + warp, j = blockIdx.y, t = blockIdx.z;
    if (f >= F) return;
    pdl_wait();
    if (!ZLM_CHK(idx + (size_t)t * top + j, 4) || !ZLM_CHK(wgt + (size_t)t * top + j, 4)) return;
    const int e = idx[(size_t)t * top + j];
    const float w = wgt[(size_t)t * top + j];
    if (e >= n_real) return;                 // an identity expert: nothing to multiply (moe_down adds its input)
    const TA* xr = x + (size_t)t * x_stride;
    const bool vec = rows_vectorise(Wup, xr, K, (size_t)K, (size_t)x_stride);
    float a;
    if (act_kind == 0) {
        const float z = warp_dot(Wup + ((size_t)e * F + f) * K, xr, K, lane, vec);
        a = scale_input ? relu2(w * z) : w * relu2(z);
    } else {
        // gated: the expert's rows are [gate | up], in groups of 8 gate rows and the 8 matching up rows (act_kind 2:
        // the layout of the products with a fused gate) or as two halves (act_kind 1)
        const size_t rg = act_kind == 2 ? (size_t)(f / 8) * 16 + f % 8 : (size_t)f;
        const size_t ru = act_kind == 2 ? rg + 8 : (size_t)F + f;
        float zg = warp_dot(Wup + ((size_t)e * 2 * F + rg) * K, xr, K, lane, vec);
        float zu = warp_dot(Wup + ((size_t)e * 2 * F + ru) * K, xr, K, lane, vec);
        if (scale_input) { zg *= w; zu *= w; }
        a = zg / (1.0f + expf(-zg)) * zu;
        if (!scale_input) a *= w;
    }
    if (lane == 0 && ZLM_CHK(act + ((size_t)t * top + j) * F + f, sizeof(TA)))
        act[((size_t)t * top + j) * F + f] = from_f32<TA>(a);
}

// stream[t, n] += sum_j Wdown[idx[t, j]][n, :] . act[t, j, :];  grid (ceil(N / MOE_WARPS), T)
template <typename TA>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_down_kernel(float* __restrict__ stream, const TA* __restrict__ act, const TA* __restrict__ Wdown,
                const int* __restrict__ idx, int top, int F, int N, int n_real, const TA* __restrict__ x, int x_stride,
                const float* __restrict__ wgt) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * MOE_WARPS + warp, t = blockIdx.y;
    if (n >= N) return;
    pdl_wait();
    float sum = 0.f;
    for (int j = 0; j < top; ++j) {
        if (!ZLM_CHK(idx + (size_t)t * top + j, 4)) continue;
        const int e = idx[(size_t)t * top + j];
        if (e >= n_real) {
            // an identity expert gives back its input, times the choice's weight
            if (x && ZLM_CHK(wgt + (size_t)t * top + j, 4) && ZLM_CHK(x + (size_t)t * x_stride + n, sizeof(TA)))
                sum += wgt[(size_t)t * top + j] * to_f32(x[(size_t)t * x_stride + n]);
            continue;
        }
        const TA* wr = Wdown + ((size_t)e * N + n) * F;
        const TA* ar = act + ((size_t)t * top + j) * F;
        sum += warp_dot(wr, ar, F, lane, rows_vectorise(Wdown, act, F, (size_t)F, (size_t)F));
    }
    if (lane == 0 && ZLM_CHK(stream + (size_t)t * N + n, 4)) stream[(size_t)t * N + n] += sum;
}

// act_kind 0: relu(z)^2 of one matrix [E][F][K]; 1: silu(gate) * up of [E][2F][K], gate rows then up rows; 2: the same
// with the rows in groups of 8 gate and 8 up.  n_real: experts from this index on are identity experts (no matrices).
extern "C" int zlm_moe_up(void* act, const void* x, int x_stride, const void* Wup, const int* idx, const float* wgt,
                          int dtype, int T, int top, int F, int K, int scale_input, int act_kind, int n_real,
                          cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(act_kind >= 0 && act_kind <= 2 && (act_kind != 2 || F % 8 == 0), "moe_up: activation %d with F=%d", act_kind, F);
    ZLM_REQUIRE(T <= 65535 && top > 0 && top <= 65535 && F > 0 && K > 0, "moe_up: bad sizes T=%d top=%d F=%d K=%d", T, top, F, K);
    dim3 grid((F + MOE_WARPS - 1) / MOE_WARPS, top, T);
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(moe_up_kernel<float>, grid, MOE_WARPS * 32, 0, st, (float*)act, (const float*)x, x_stride,
                   (const float*)Wup, idx, wgt, top, F, K, scale_input, act_kind, n_real);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(moe_up_kernel<__nv_bfloat16>, grid, MOE_WARPS * 32, 0, st, (__nv_bfloat16*)act, (const __nv_bfloat16*)x,
                   x_stride, (const __nv_bfloat16*)Wup, idx, wgt, top, F, K, scale_input, act_kind, n_real);
    else
        ZLM_REQUIRE(false, "moe_up: unsupported dtype %d", dtype);
    return zlm_check_launch("moe_up");
}

// n_real, x, wgt: a choice of an expert from n_real on adds wgt * x[t] (an identity expert); x null: there are none
extern "C" int zlm_moe_down(float* stream, const void* act, const void* Wdown, const int* idx, int dtype, int T, int top,
                            int F, int N, int n_real, const void* x, int x_stride, const float* wgt, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(T <= 65535 && top > 0 && F > 0 && N > 0, "moe_down: bad sizes T=%d top=%d F=%d N=%d", T, top, F, N);
    dim3 grid((N + MOE_WARPS - 1) / MOE_WARPS, T);
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(moe_down_kernel<float>, grid, MOE_WARPS * 32, 0, st, stream, (const float*)act, (const float*)Wdown, idx,
                   top, F, N, n_real, (const float*)x, x_stride, wgt);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(moe_down_kernel<__nv_bfloat16>, grid, MOE_WARPS * 32, 0, st, stream, (const __nv_bfloat16*)act,
                   (const __nv_bfloat16*)Wdown, idx, top, F, N, n_real, (const __nv_bfloat16*)x, x_stride, wgt);
    else
        ZLM_REQUIRE(false, "moe_down: unsupported dtype %d", dtype);
    return zlm_check_launch("moe_down");
}

// ---------------------------------------------------------------------------- activation with a row scale
template <typename TA>
__global__ void act_scale_kernel(TA* __restrict__ out, const TA* __restrict__ u, const float* __restrict__ s, int T, int F) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)T * F;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / F;
        if (!ZLM_CHK(u + e, sizeof(TA)) || !ZLM_CHK(out + e, sizeof(TA)) || (s && !ZLM_CHK(s + t, 4))) continue;
        out[e] = from_f32<TA>(relu2(to_f32(u[e])) * (s ? s[t] : 1.0f));
    }
}

extern "C" int zlm_relu2_scale(void* out, const void* u, const float* s, int dtype, int T, int F, cudaStream_t st) {
    if (T == 0 || F == 0) return ZLM_OK;
    const size_t n = (size_t)T * F;
    int blocks = (int)((n + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == ZLM_DTYPE_F32)
        zlm_launch(act_scale_kernel<float>, blocks, 256, 0, st, (float*)out, (const float*)u, s, T, F);
    else if (dtype == ZLM_DTYPE_BF16)
        zlm_launch(act_scale_kernel<__nv_bfloat16>, blocks, 256, 0, st, (__nv_bfloat16*)out, (const __nv_bfloat16*)u, s, T, F);
    else
        ZLM_REQUIRE(false, "relu2_scale: unsupported dtype %d", dtype);
    return zlm_check_launch("relu2_scale");
}

ZLM_TRANSLATION_UNIT(moe)
