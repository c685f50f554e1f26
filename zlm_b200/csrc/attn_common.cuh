// Helpers shared by the tensor-core attention kernels (decode and prefill):
// cp.async staging, ldmatrix, the bf16 m16n8k16 product, and the swizzled layout
// of a [64][head_dim] tile in shared memory.
#pragma once
#include "common.cuh"

__device__ __forceinline__ void dec_cp_async16(void* smem, const void* gmem) {
    if (!ZLM_CHK(gmem, 16)) return;
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void dec_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void dec_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void dec_ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void dec_ldsm4t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void dec_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&v;
}

// What a mixer may ask of the attention kernels beyond the scale and the window.
//   chunk    > 0: a query sees only the keys of its own chunk of that many positions, counted from position 0
//   softcap  > 0: scores become softcap * tanh(score * scale / softcap)
//   sinks    one number per query head whose exponential joins the softmax's denominator without a value
//            (null with the flag `sink` set: the number is 0)
//   v_share  that many neighbouring key heads read one value head: a page is [nkv key heads | nkv / v_share value
//            heads] of [ZLM_PAGE][hd] each (1: the ordinary [K | V] of nkv heads each)
struct AttnOpts {
    int chunk;
    float softcap;
    const float* sinks;
    int v_share;
};
static inline AttnOpts attn_no_opts() { return AttnOpts{0, 0.f, nullptr, 1}; }

// the first key that the query at `pos` reads
__device__ __forceinline__ int attn_first_key(int pos, int window, int chunk) {
    int lo = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
    if (chunk > 0) lo = max(lo, pos - pos % chunk);
    return lo;
}

// a raw dot product as a base-2 exponent: dot * scale * log2(e), capped first where the mixer asks for it
// (tanh through one exponential: 1 - 2 / (e^{2x} + 1), absolute error of a few 1e-7 of the cap)
__device__ __forceinline__ float attn_score_log2(float dot, float scale_log2, float softcap) {
    if (softcap <= 0.f) return dot * scale_log2;
    const float x = dot * scale_log2 / softcap;               // y = dot * scale / softcap = x / log2(e): e^{2y} = 2^{2x}
    const float th = 1.0f - __fdividef(2.0f, exp2f(2.0f * x) + 1.0f);
    return softcap * 1.4426950408889634f * th;
}

// a tile's raw dot products as base-2 exponents, all at once: whether there is a cap is asked once (every thread of
// a launch answers alike), so a kernel without one pays a multiplication a score and nothing else
template <int NT> __device__ __forceinline__ void attn_scores_log2(float (&s)[NT][4], float scale_log2, float softcap) {
    if (softcap > 0.f) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = attn_score_log2(s[nt][e], scale_log2, softcap);
    } else {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] *= scale_log2;
    }
}

// the running maximum a row starts from (base-2 exponent) when the softmax has a sink
__device__ __forceinline__ float attn_sink_log2(const float* sinks, int head) {
    return (sinks && ZLM_CHK(sinks + head, 4)) ? sinks[head] * 1.4426950408889634f : 0.f;
}

// element offset of (row, 16-byte chunk) inside a [64][HD] tile; rows of 128 bytes
// or more are swizzled so that ldmatrix reads 8 rows without bank conflicts
template <int HD> __device__ __forceinline__ int tile_off(int row, int chunk) {
    constexpr int SW = (HD % 64 == 0) ? 7 : 0;
    return row * HD + ((chunk ^ (row & SW)) << 3);
}

