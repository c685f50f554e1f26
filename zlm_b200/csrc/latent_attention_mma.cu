// Latent attention over the paged bf16 records on the warp-level tensor cores, for decode steps and
// for prompts.  A record is [c (r) | kr (dr)], D = r + dr; a query row is [q' (r) | rotated part (dr)];
// every head reads the same records, so the 16 rows of a tile are 16 heads of one token and a page
// of records, staged once in shared memory, serves as keys (all D columns) and as values (the
// first r columns).
//
// grid (token group, head tile, split).  A block has QT groups of 4 or 8 warps; group i works on token
// t0 + i, and all groups share the staged pages (tokens of one block that belong to different
// sequences are walked one sequence after the other).  Per page of 64 records a group computes
//   S = Q K^T     each warp 16 keys (8 in groups of 8 warps), Q fragments from shared memory (D is too wide for registers)
//   the page's row maxima across the four warps, P = exp2(S - m) as bf16 in shared memory
//   O += P V      each warp all 64 keys for its share of the r value columns (units of 16 columns
//                 dealt round-robin), so no warp holds more than 16 x 16 NU accumulators
// with an fp32 running maximum and sum per head.  Pages come by cp.async, two stages.  With more than
// one split (decode steps) the (max, sum, O) of a split go to scratch and the decode attention's
// combine kernel merges them in a fixed order.  Options: `chunk` (a query reads only the records of its own chunk of
// that many positions, counted from position 0) and `sinks` (a number per head whose exponential joins the softmax's
// denominator without a value).
#include "common.cuh"
#include "attn_common.cuh"

#define LM_PAD 8               // elements of padding per shared-memory row: rows 16 bytes apart in the banks

// GW: warps of a group (4: each takes 16 of a page's keys, two score tiles; 8: 8 keys, one score tile, and half
// as many value columns a warp, for sizes whose shared memory leaves room for few tokens a block: twice the
// warps an SM holds)
template <int NU, int QT, int GW>
__global__ void __launch_bounds__(GW * 32 * QT)
latent_mma_kernel(__nv_bfloat16* __restrict__ out, int out_stride, const __nv_bfloat16* __restrict__ q, int q_stride,
                  const __nv_bfloat16* __restrict__ pool, const int* __restrict__ block_table, int table_stride,
                  const int* __restrict__ token_pos, const int* __restrict__ token_slot, int T, int H, int r, int dr,
                  float scale_log2, int window, int splits, int per, float* __restrict__ part_o,
                  float* __restrict__ part_ml, int fresh, int chunk, const float* __restrict__ sinks) {
    constexpr int GT = GW * 32;                  // threads of a group
    constexpr int NTK = 8 / GW;                  // score tiles (of 8 keys) a warp takes of a page
    constexpr int WK = 8 * NTK;                  // keys a warp takes of a page
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int D = r + dr, DS = D + LM_PAD, PS = ZLM_PAGE + LM_PAD;
    const int KS = D / 16, NV = r / 16;
    __nv_bfloat16* Rs = (__nv_bfloat16*)smem_raw;                         // [2][64][DS] the staged pages
    __nv_bfloat16* Qs = Rs + 2 * ZLM_PAGE * DS;                           // [QT][16][DS]
    __nv_bfloat16* Ps = Qs + QT * 16 * DS;                                // [QT][16][PS]
    float* smax = (float*)(Ps + QT * 16 * PS);                            // [QT][GW][16], later the warps' sums

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int grp = warp / GW, wq = warp % GW;
    const int g = lane >> 2, qd = lane & 3;
    // prompts: the last tokens of a sequence walk the most pages, so their blocks go first (blocks start in
    // the order of their index) and the short ones fill in behind them
    const int t0 = (QT > 1 ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x) * QT, htile = blockIdx.y, split = blockIdx.z;
    const GroupSync gsync{1 + grp, GT};
    pdl_launch_dependents();

    const int my_t = t0 + grp;
    const bool have = my_t < T;
    int my_pos = 0, my_slot = -1;
    if (have && ZLM_CHK(token_pos + my_t, 4) && ZLM_CHK(token_slot + my_t, 4)) {
        my_pos = token_pos[my_t];
        my_slot = token_slot[my_t];
    }
    const int my_start = attn_first_key(my_pos, window, chunk);

    auto load_page = [&](const int* pages, int p, int stage) {
        if (!ZLM_CHK(pages + p, 4)) return;
        const __nv_bfloat16* src = pool + (size_t)pages[p] * ZLM_PAGE * D;
        __nv_bfloat16* dst = Rs + (size_t)stage * ZLM_PAGE * DS;
        const int CH = D / 8;
        for (int id = tid; id < ZLM_PAGE * CH; id += GT * QT) {
            const int row = id / CH, c = id - row * CH;
            dec_cp_async16(dst + row * DS + c * 8, src + (size_t)row * D + c * 8);
        }
    };

    float o[2 * NU][4];
#pragma unroll
    for (int i = 0; i < 2 * NU; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;          // rows g and g + 8
    if (sinks && split == 0) {
        // exp(sinks[head]) joins the row's sum without a value, once per (token, head): every warp of the group
        // starts from it as the running maximum, one lane of one warp counts it
        const int h0 = htile * 16 + g, h1 = h0 + 8;
        m0 = h0 < H ? attn_sink_log2(sinks, h0) : 0.f;
        m1 = h1 < H ? attn_sink_log2(sinks, h1) : 0.f;
        if (wq == 0 && qd == 0) l0 = l1 = 1.f;
    }
    bool q_loaded = false, waited = false;

    // the block's tokens, one run of equal slots after the other (a decode step: one token, one run)
    for (int lead = 0; lead < QT && t0 + lead < T; ++lead) {
        if (!ZLM_CHK(token_slot + t0 + lead, 4) || !ZLM_CHK(token_pos + t0 + lead, 4)) break;
        const int slot = token_slot[t0 + lead];
        if (lead > 0 && token_slot[t0 + lead - 1] == slot) continue;       // belongs to the run before
        int lo = 0x7fffffff, hi = -1;
        for (int i = lead; i < QT && t0 + i < T && token_slot[t0 + i] == slot; ++i) {
            const int p = token_pos[t0 + i];
            lo = min(lo, attn_first_key(p, window, chunk));
            hi = max(hi, p);
        }
        const bool mine = have && my_slot == slot;
        const int* pages = block_table + (size_t)slot * table_stride;
        const int page_lo = lo / ZLM_PAGE, page_hi = hi / ZLM_PAGE + 1;
        const int p_begin = page_lo + split * per;
        const int p_end = min(page_hi, p_begin + per);
        if (p_begin >= p_end) continue;                                     // (the combine kernel skips this split too)

        // pages that hold positions of earlier steps only do not wait for the kernel before this one
        const int old_pages = (QT == 1 && fresh > 0) ? max(0, hi + 1 - fresh) / ZLM_PAGE : 0;
        const bool early0 = lead == 0 && p_begin < old_pages;
        const bool early1 = early0 && p_begin + 1 < p_end && p_begin + 1 < old_pages;
        if (early0) {
            load_page(pages, p_begin, 0);
            dec_commit();
            if (early1) {
                load_page(pages, p_begin + 1, 1);
                dec_commit();
            }
        }
        if (!waited) {
            pdl_wait();
            waited = true;
        }
        if (!early0) {
            load_page(pages, p_begin, 0);
            dec_commit();
        }
        if (!early1) {
            if (p_begin + 1 < p_end) load_page(pages, p_begin + 1, 1);
            dec_commit();
        }
        if (!q_loaded) {
            // the 16 heads of this tile for every group's token (zero rows beyond the last head or token)
            const int CH = D / 8;
            for (int id = tid; id < QT * 16 * CH; id += GT * QT) {
                const int gi = id / (16 * CH), rem = id - gi * 16 * CH, row = rem / CH, c = rem - row * CH;
                const int head = htile * 16 + row, t = t0 + gi;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                const __nv_bfloat16* src = q + (size_t)t * q_stride + (size_t)head * D + c * 8;
                if (t < T && head < H && ZLM_CHK(src, 16)) v = *(const uint4*)src;
                *(uint4*)(Qs + ((size_t)gi * 16 + row) * DS + c * 8) = v;
            }
            q_loaded = true;
        }

        for (int p = p_begin; p < p_end; ++p) {
            const int stage = (p - p_begin) & 1;
            dec_wait<1>();
            __syncthreads();                         // page p (and, the first time, Q) is there
            const bool busy = mine && p * ZLM_PAGE <= my_pos && p * ZLM_PAGE + ZLM_PAGE - 1 >= my_start;   // group-uniform
            if (busy) {
                const __nv_bfloat16* rt = Rs + (size_t)stage * ZLM_PAGE * DS;
                const __nv_bfloat16* qt = Qs + (size_t)grp * 16 * DS;
                __nv_bfloat16* pt = Ps + (size_t)grp * 16 * PS;
                float* mx = smax + grp * GW * 16;
                // two chains of sums, even and odd steps of 16 columns (a product waits for the one before it in
                // its chain), added at the end
                float s[NTK][4], s2[NTK][4];
#pragma unroll
                for (int i = 0; i < NTK; ++i)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[i][e] = s2[i][e] = 0.f;
                const int mi = lane >> 3;
                const int a_row = (lane & 7) + (mi & 1) * 8, a_chunk = mi >> 1;
                if (GW == 4) {
                    const int b_row = wq * 16 + (mi >> 1) * 8 + (lane & 7), b_chunk = mi & 1;
#pragma unroll 2
                    for (int ks = 0; ks + 1 < KS; ks += 2) {
                        unsigned a[4], c[4], b00, b01, b10, b11, d00, d01, d10, d11;
                        dec_ldsm4(a[0], a[1], a[2], a[3], qt + a_row * DS + (ks * 2 + a_chunk) * 8);
                        dec_ldsm4(b00, b01, b10, b11, rt + b_row * DS + (ks * 2 + b_chunk) * 8);
                        dec_ldsm4(c[0], c[1], c[2], c[3], qt + a_row * DS + (ks * 2 + 2 + a_chunk) * 8);
                        dec_ldsm4(d00, d01, d10, d11, rt + b_row * DS + (ks * 2 + 2 + b_chunk) * 8);
                        dec_mma(s[0], a, b00, b01);
                        dec_mma(s[NTK - 1], a, b10, b11);
                        dec_mma(s2[0], c, d00, d01);
                        dec_mma(s2[NTK - 1], c, d10, d11);
                    }
                    if (KS & 1) {
                        const int ks = KS - 1;
                        unsigned a[4], b00, b01, b10, b11;
                        dec_ldsm4(a[0], a[1], a[2], a[3], qt + a_row * DS + (ks * 2 + a_chunk) * 8);
                        dec_ldsm4(b00, b01, b10, b11, rt + b_row * DS + (ks * 2 + b_chunk) * 8);
                        dec_mma(s[0], a, b00, b01);
                        dec_mma(s[NTK - 1], a, b10, b11);
                    }
                } else {
                    // 8 keys a warp: one load brings the key fragments of two steps (columns ks*16 .. ks*16+31)
                    const int b_row = wq * 8 + (lane & 7);
#pragma unroll 2
                    for (int ks = 0; ks + 1 < KS; ks += 2) {
                        unsigned a[4], c[4], b0, b1, b2, b3;
                        dec_ldsm4(a[0], a[1], a[2], a[3], qt + a_row * DS + (ks * 2 + a_chunk) * 8);
                        dec_ldsm4(c[0], c[1], c[2], c[3], qt + a_row * DS + (ks * 2 + 2 + a_chunk) * 8);
                        dec_ldsm4(b0, b1, b2, b3, rt + b_row * DS + (ks * 2 + mi) * 8);
                        dec_mma(s[0], a, b0, b1);
                        dec_mma(s2[0], c, b2, b3);
                    }
                    if (KS & 1) {
                        const int ks = KS - 1;
                        unsigned a[4], b0, b1, b2, b3;
                        dec_ldsm4(a[0], a[1], a[2], a[3], qt + a_row * DS + (ks * 2 + a_chunk) * 8);
                        dec_ldsm4(b0, b1, b2, b3, rt + b_row * DS + (ks * 2 + (mi & 1)) * 8);      // (the last two repeat the first)
                        dec_mma(s[0], a, b0, b1);
                    }
                }
#pragma unroll
                for (int i = 0; i < NTK; ++i)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[i][e] += s2[i][e];
                const int kbase = p * ZLM_PAGE + wq * WK;
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < NTK; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = kbase + nt * 8 + qd * 2 + e;
                        const bool ok = key <= my_pos && key >= my_start;
                        s[nt][e] = ok ? s[nt][e] * scale_log2 : -INFINITY;
                        s[nt][2 + e] = ok ? s[nt][2 + e] * scale_log2 : -INFINITY;
                        mx0 = fmaxf(mx0, s[nt][e]);
                        mx1 = fmaxf(mx1, s[nt][2 + e]);
                    }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                if (qd == 0) {
                    mx[wq * 16 + g] = mx0;
                    mx[wq * 16 + g + 8] = mx1;
                }
                gsync.sync();
                float pm0 = -INFINITY, pm1 = -INFINITY;
#pragma unroll
                for (int w = 0; w < GW; ++w) {
                    pm0 = fmaxf(pm0, mx[w * 16 + g]);
                    pm1 = fmaxf(pm1, mx[w * 16 + g + 8]);
                }
                const float mn0 = fmaxf(m0, pm0), mn1 = fmaxf(m1, pm1);        // finite: the page has a key in reach
                const float a0 = m0 == -INFINITY ? 0.f : exp2f(m0 - mn0);
                const float a1 = m1 == -INFINITY ? 0.f : exp2f(m1 - mn1);
                m0 = mn0;
                m1 = mn1;
                float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
                for (int nt = 0; nt < NTK; ++nt) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        s[nt][e] = s[nt][e] == -INFINITY ? 0.f : exp2f(s[nt][e] - mn0);
                        s[nt][2 + e] = s[nt][2 + e] == -INFINITY ? 0.f : exp2f(s[nt][2 + e] - mn1);
                        ps0 += s[nt][e];
                        ps1 += s[nt][2 + e];
                    }
                    const int col = wq * WK + nt * 8 + qd * 2;
                    *(unsigned*)(pt + g * PS + col) = pack_bf16(s[nt][0], s[nt][1]);
                    *(unsigned*)(pt + (g + 8) * PS + col) = pack_bf16(s[nt][2], s[nt][3]);
                }
                l0 = l0 * a0 + ps0;
                l1 = l1 * a1 + ps1;
#pragma unroll
                for (int i = 0; i < 2 * NU; ++i) {
                    o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1;
                }
                gsync.sync();                        // P of all the group's warps is there
                const int v_row = (mi & 1) * 8 + (lane & 7), v_chunk = mi >> 1;
#pragma unroll
                for (int kk = 0; kk < ZLM_PAGE / 16; ++kk) {
                    unsigned a[4];
                    dec_ldsm4(a[0], a[1], a[2], a[3], pt + a_row * PS + (kk * 2 + a_chunk) * 8);
#pragma unroll
                    for (int j = 0; j < NU; ++j) {
                        const int u = wq + GW * j;
                        if (u < NV) {
                            unsigned b0, b1, b2, b3;
                            dec_ldsm4t(b0, b1, b2, b3, rt + (kk * 16 + v_row) * DS + (u * 2 + v_chunk) * 8);
                            dec_mma(o[2 * j], a, b0, b1);
                            dec_mma(o[2 * j + 1], a, b2, b3);
                        }
                    }
                }
            }
            __syncthreads();                         // every warp is done with this stage
            if (p + 2 < p_end) load_page(pages, p + 2, stage);
            dec_commit();
        }
        dec_wait<0>();
    }
    if (!waited) pdl_wait();
    __syncthreads();
    if (!have || my_slot < 0) return;

    // the group's warps' sums of a row in a fixed order
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* sl = smax + grp * GW * 16;
    if (qd == 0) {
        sl[wq * 16 + g] = l0;
        sl[wq * 16 + g + 8] = l1;
    }
    gsync.sync();
    float L0 = 0.f, L1 = 0.f;
#pragma unroll
    for (int w = 0; w < GW; ++w) {
        L0 += sl[w * 16 + g];
        L1 += sl[w * 16 + g + 8];
    }
    const int h0 = htile * 16 + g, h1 = h0 + 8;
#pragma unroll
    for (int j = 0; j < NU; ++j) {
        const int u = wq + GW * j;
        if (u >= NV) continue;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int col = u * 16 + half * 8 + qd * 2;
            const float* ov = o[2 * j + half];
            if (splits == 1) {
                if (h0 < H && ZLM_CHK(out + (size_t)my_t * out_stride + (size_t)h0 * r + col, 4))
                    *(unsigned*)(out + (size_t)my_t * out_stride + (size_t)h0 * r + col) = pack_bf16(ov[0] / L0, ov[1] / L0);
                if (h1 < H && ZLM_CHK(out + (size_t)my_t * out_stride + (size_t)h1 * r + col, 4))
                    *(unsigned*)(out + (size_t)my_t * out_stride + (size_t)h1 * r + col) = pack_bf16(ov[2] / L1, ov[3] / L1);
            } else {
                if (h0 < H) {
                    float* po = part_o + (((size_t)my_t * H + h0) * splits + split) * r + col;
                    if (ZLM_CHK(po, 8)) { po[0] = ov[0]; po[1] = ov[1]; }
                }
                if (h1 < H) {
                    float* po = part_o + (((size_t)my_t * H + h1) * splits + split) * r + col;
                    if (ZLM_CHK(po, 8)) { po[0] = ov[2]; po[1] = ov[3]; }
                }
            }
        }
    }
    if (splits > 1 && wq == 0 && qd == 0) {
        if (h0 < H) {
            float* ml = part_ml + (((size_t)my_t * H + h0) * splits + split) * 2;
            if (ZLM_CHK(ml, 8)) { ml[0] = m0; ml[1] = L0; }      // (-inf, 0) if the split held no key of this token
        }
        if (h1 < H) {
            float* ml = part_ml + (((size_t)my_t * H + h1) * splits + split) * 2;
            if (ZLM_CHK(ml, 8)) { ml[0] = m1; ml[1] = L1; }
        }
    }
}

// the decode attention's combine kernel (attention_decode.cu) merges the splits
extern "C" int zlm_attention_decode_combine_chunk(void* out, int out_stride, const float* part_o, const float* part_ml,
                                                  const int* token_pos, int T, int nq, int hd, int splits, int per,
                                                  int window, int chunk, cudaStream_t st);

static size_t latent_mma_smem(int D, int QT) {
    const size_t DS = D + LM_PAD, PS = ZLM_PAGE + LM_PAD;
    return (2 * ZLM_PAGE * DS + (size_t)QT * 16 * DS + (size_t)QT * 16 * PS) * 2 + (size_t)QT * 8 * 16 * 4;
}

// 1 if the tensor-core kernel takes the shape (else the caller uses the plain kernel)
extern "C" int zlm_latent_attention_mma_supported(int H, int r, int dr) {
    return (H > 0 && r >= 16 && r % 16 == 0 && dr % 16 == 0 && r <= 512 && latent_mma_smem(r + dr, 1) <= 220 * 1024) ? 1 : 0;
}

// blocks of the one-token form that an SM holds at a time (its pages of records are large: shared memory decides)
extern "C" int zlm_latent_attention_mma_blocks_per_sm(int r, int dr) {
    const size_t one = latent_mma_smem(r + dr, 1) + 1024;
    const int n = (int)((size_t)228 * 1024 / one);
    return n < 1 ? 1 : (n > 8 ? 8 : n);
}

// tokens a block takes in a step of many tokens per sequence: as many as the shared memory holds
extern "C" int zlm_latent_attention_mma_tokens(int r, int dr) {
    const int D = r + dr;
    if (latent_mma_smem(D, 4) <= 220 * 1024) return 4;
    if (latent_mma_smem(D, 2) <= 220 * 1024) return 2;
    return 1;
}

template <int NU, int QT, int GW>
static int launch_latent_mma(void* out, int out_stride, const void* q, int q_stride, const void* pool,
                             const int* block_table, int table_stride, const int* token_pos, const int* token_slot,
                             int T, int H, int r, int dr, float scale, int window, int splits, int per, float* part_o,
                             float* part_ml, int fresh, int chunk, const float* sinks, cudaStream_t st) {
    const size_t smem = latent_mma_smem(r + dr, QT);
    auto kern = latent_mma_kernel<NU, QT, GW>;
    static size_t reserved[64] = {};
    size_t& have = reserved[zlm_device_index()];
    if (smem > have) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            zlm_set_error("latent_attention_mma: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return ZLM_ERR_CUDA;
        }
        have = smem;
    }
    dim3 grid((T + QT - 1) / QT, (H + 15) / 16, splits);
    zlm_launch(kern, grid, dim3(GW * 32 * QT), smem, st, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,
               (const __nv_bfloat16*)pool, block_table, table_stride, token_pos, token_slot, T, H, r, dr,
               scale * 1.4426950408889634f, window, splits, per, part_o, part_ml, fresh, chunk, sinks);
    int rc = zlm_check_launch("latent_attention_mma");
    if (rc) return rc;
    if (splits > 1)
        rc = zlm_attention_decode_combine_chunk(out, out_stride, part_o, part_ml, token_pos, T, H, r, splits, per, window,
                                                chunk, st);
    return rc;
}

// tokens_per_block 1: a decode step (splits of `per` pages each; scratch part_o T*H*splits*r floats, part_ml
// T*H*splits*2); 2 or 4: prompts and portions (splits must be 1; `per` covers the longest sequence).
extern "C" int zlm_latent_attention_mma(void* out, int out_stride, const void* q, int q_stride, const void* pool,
                                        const int* block_table, int table_stride, const int* token_pos,
                                        const int* token_slot, int T, int H, int r, int dr, float scale, int window,
                                        int tokens_per_block, int splits, int per, float* part_o, float* part_ml,
                                        int fresh, int chunk, const float* sinks, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(chunk >= 0, "latent_attention_mma: chunk=%d", chunk);
    ZLM_REQUIRE(zlm_latent_attention_mma_supported(H, r, dr), "latent_attention_mma: heads=%d kv_rank=%d rot_dim=%d is not a "
                "shape this kernel takes", H, r, dr);
    ZLM_REQUIRE(splits >= 1 && splits <= 1024 && per >= 1 && (splits == 1 || tokens_per_block == 1),
                "latent_attention_mma: splits=%d of %d pages, %d tokens a block", splits, per, tokens_per_block);
    ZLM_REQUIRE(splits == 1 || (part_o && part_ml), "latent_attention_mma: scratch missing for %d splits", splits);
    ZLM_REQUIRE((uintptr_t)q % 16 == 0 && (q_stride * 2) % 16 == 0 && ((r + dr) * 2) % 16 == 0 && (uintptr_t)out % 4 == 0 &&
                out_stride % 2 == 0, "latent_attention_mma: q must be 16-byte aligned, out 4-byte aligned");
    ZLM_REQUIRE((H + 15) / 16 <= 65535 && splits <= 65535, "latent_attention_mma: too many head tiles or splits");
    // groups of 8 warps where a block has one or two tokens (large records: twice the warps an SM holds, half the
    // value columns a warp); groups of 4 where four tokens fit
    const int nu4 = ((r / 16) + 3) / 4, nu8 = ((r / 16) + 7) / 8;
#define ZLM_LM(NU, QT, GW)                                                                                           \
    return launch_latent_mma<NU, QT, GW>(out, out_stride, q, q_stride, pool, block_table, table_stride, token_pos,  \
                                         token_slot, T, H, r, dr, scale, window, splits, per, part_o, part_ml, fresh, chunk, \
                                         sinks, st)
#define ZLM_LM_8(QT)                              \
    do {                                          \
        if (nu8 <= 1) ZLM_LM(1, QT, 8);           \
        if (nu8 <= 2) ZLM_LM(2, QT, 8);           \
        ZLM_LM(4, QT, 8);                         \
    } while (0)
    if (tokens_per_block == 1) ZLM_LM_8(1);
    if (tokens_per_block == 2) ZLM_LM_8(2);
    if (tokens_per_block == 4) {
        if (nu4 <= 1) ZLM_LM(1, 4, 4);
        if (nu4 <= 2) ZLM_LM(2, 4, 4);
        if (nu4 <= 4) ZLM_LM(4, 4, 4);
        ZLM_LM(8, 4, 4);
    }
#undef ZLM_LM_8
#undef ZLM_LM
    ZLM_REQUIRE(false, "latent_attention_mma: %d tokens a block (1, 2 or 4)", tokens_per_block);
}

ZLM_TRANSLATION_UNIT(latent_attention_mma)
