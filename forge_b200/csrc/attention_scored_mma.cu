// Tensor-core form (bf16 operands, fp32 sums) of the causal attention with shaped scores, for prompt portions and single
// tokens alike; see attention_scored.cu for the definition and the cache layout.
//
// Every (query head, map) is an ordinary one-pass attention of its own (running maximum and sum in registers) over the keys
// of ITS map and the values of its key/value head.  A CTA of four warps takes a tile of up to 64 rows = tokens x the query
// heads of ONE key/value head, for ONE map (consecutive tokens of one request; a single token brings H/G rows), one chunk
// of VC value columns, and walks the keys in tiles of 64 positions that start at multiples of 64.  With one map the result
// goes out in bfloat16 at once; with two, each map leaves its normalised output in fp32 and a second kernel takes
// a_1 - lambda a_2, divides by the root mean square and scales.  The distance term is taken off the scores in fp32 before
// the softmax (with the fast base-2 logarithm; the 32-bit kernel of attention_scored.cu uses log1pf).  mma.sync m16n8k16 (the legacy tensor path): S = Q K^T with K rows as the column-major operand, O += P V with
// V through ldmatrix.trans; a softmax weight is the value product's operand as two bfloat16 numbers (16 bits of mantissa).
#include "common.cuh"
#include "checks.cuh"

namespace {

constexpr int BM = 64, BN = 64, kThreads = 128, kPad = 8;
constexpr int kMmaSmemLimit = 200 * 1024;

// The first position that position `pos` sees (window: i - j < window; chunk: the same chunk of positions; 0 = no such limit).
__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
    int lo = 0;
    if (window > 0) lo = max(lo, pos - window + 1);
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);
    return lo;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory without a stop in registers; ok == false writes zeros instead
__device__ __forceinline__ void copy16_async(void* dst, const void* src, bool ok) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = ok ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float ex2(float x) {          // 2^x, relative error 2^-22; ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// tanh(x) = 1 - 2 / (e^(2x) + 1) from the approximate exponential and reciprocal: absolute error about 2e-7 (and exactly +-1
// far out), which a score from bfloat16 operands does not see; the kernel of fp32 arithmetic keeps tanhf
__device__ __forceinline__ float tanh_fast(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(ex2(x * 2.8853900817779268f) + 1.0f));
    return fmaf(-2.0f, r, 1.0f);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// M == 1 and nsplit == 1: out bf16 [T, H, E] (times out_scale).  Otherwise u fp32 [nsplit, T, H, M, E]: normalised with
// nsplit == 1; with nsplit > 1 (steps of single tokens: a request's key tiles are dealt out to nsplit CTAs in runs) each run
// leaves its sums as they are, beside the row's maximum (in units of log2 e) and sum in part_ml [nsplit, T, H, M, 2].
template <int VC, bool SPLIT>
__global__ void __launch_bounds__(kThreads)
scored_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache, const int32_t* __restrict__ block_table,
                  const int32_t* __restrict__ tok_req, const int32_t* __restrict__ positions, const int32_t* __restrict__ tile_t0,
                  const int32_t* __restrict__ tile_n, const float* __restrict__ r1, const float* __restrict__ r2, float* __restrict__ u,
                  __nv_bfloat16* __restrict__ out, float* __restrict__ part_ml, int nsplit_given, int T, int qrows, int H, int G, int M, int D, int E, int page_size, long long page_stride,
                  int max_pages, float scale, float out_scale, long long out_ld, int window, int chunk, float softcap) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int nsplit = SPLIT ? nsplit_given : 1;          // (a prompt's kernel is compiled without the dealing out)
    // the last tiles of a prompt see the most keys: they start first, so that the short ones fill the grid's tail
    const int tile = gridDim.x / nsplit - 1 - blockIdx.x / nsplit, sp = blockIdx.x % nsplit, c = blockIdx.y / M, mp = blockIdx.y % M, v0 = blockIdx.z * VC;
    const int t0 = tile_t0 ? tile_t0[tile] : tile;
    const int nq = tile_n ? tile_n[tile] : 1;
    if (!FORGE_TOKEN_OK(t0) || !FORGE_TOKEN_OK(t0 + nq - 1)) return;
    const int Gq = H / G, rows = nq * Gq, KD = M * D;
    const int pos0 = positions[t0], pos_last = pos0 + nq - 1;
    const int32_t* table = block_table + (size_t)tok_req[t0] * max_pages;
    const int DP = D + kPad, VP = VC + kPad;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [qrows][D + 8]
    const int stage = BN * (DP + VP);                                     // elements of one buffer: a key tile and a value tile
    __nv_bfloat16* Ks = Qs + qrows * DP;                                  // 2 x [BN][D + 8]
    __nv_bfloat16* Vs = Ks + BN * DP;                                     // 2 x [BN][VC + 8], each behind its key tile
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    // queries: row r = token t0 + r / Gq, head c * Gq + r % Gq, map mp
    const int dchunks = D >> 3;
    for (int i = tid; i < qrows * dchunks; i += kThreads) {
        const int r = i / dchunks, ch = i % dchunks;
        uint4 val = zero4;
        if (r < rows)
            val = *reinterpret_cast<const uint4*>(q + (((size_t)(t0 + r / Gq) * H + c * Gq + r % Gq) * M + mp) * D + ch * 8);
        *reinterpret_cast<uint4*>(Qs + r * DP + ch * 8) = val;
    }

    float oacc[VC / 8][4];
#pragma unroll
    for (int i = 0; i < VC / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
    float row_m[2] = {-INFINITY, -INFINITY}, row_l[2] = {0.f, 0.f};
    // A tile of at most 16 rows (a single token: H/G rows) would leave three warps idle: there all four warps take the same
    // 16 rows, each computes the scores again, and each takes a quarter of the value columns.
    const bool colsplit = rows <= 16;
    const int rb = colsplit ? 0 : warp;                                   // this warp's block of 16 rows
    const int ntw = colsplit ? VC / 32 : VC / 8, cb = colsplit ? warp * (VC / 4) : 0;     // its value columns: ntw blocks of 8 from cb
    const int r_lo = rb * 16 + (lane >> 2), r_hi = r_lo + 8;             // this thread's two rows
    const int pos_lo = pos0 + min(r_lo, rows - 1) / Gq, pos_hi = pos0 + min(r_hi, rows - 1) / Gq;
    const bool live_lo = r_lo < rows, live_hi = r_hi < rows;
    const int see_lo = first_visible(pos_lo, window, chunk), see_hi = first_visible(pos_hi, window, chunk);
    const int see_last = first_visible(pos_last, window, chunk);          // the tile's last token sees no earlier key than any other
    const float cap_in = softcap > 0.f ? scale / softcap : 0.f, cap_out = softcap * 1.4426950408889634f;
    const int h_lo = c * Gq + min(r_lo, rows - 1) % Gq, h_hi = c * Gq + min(r_hi, rows - 1) % Gq;
    const float r1v[2] = {r1 ? r1[h_lo] : 0.f, r1 ? r1[h_hi] : 0.f}, r2v[2] = {r1 ? r2[h_lo] : 0.f, r1 ? r2[h_hi] : 0.f};

    const int last_tile = pos_last / BN;
    constexpr float kLog2e = 1.4426950408889634f;
    const float sl2 = scale * kLog2e;                                     // scores in units of log2(e)
    const int vchunks = VC >> 3;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    const size_t v_base = (size_t)G * page_size * KD + (size_t)c * page_size * E;

    // key and value tiles go through two buffers: tile ti + 1 is on its way while tile ti is worked on.  Two threads a key row.
    const int frow = tid >> 1, fpar = tid & 1;
    auto fetch = [&](int kt, int buf) {
        const int j = kt * BN + frow;
        __nv_bfloat16* Kb = Ks + buf * stage + frow * DP;
        __nv_bfloat16* Vb = Vs + buf * stage + frow * VP;
        const __nv_bfloat16* page_base = cache;
        bool ok = false;
        if (j <= pos_last) {
            const int page = table[j >> page_shift];
            if (page >= 0 && FORGE_PAGE_OK(page)) {
                ok = true;
                page_base = cache + (size_t)page * page_stride;
            }
        }
        const int off = j & (page_size - 1);
        const __nv_bfloat16* ksrc = page_base + ((size_t)c * page_size + off) * KD + mp * D;
        for (int ch = fpar; ch < dchunks; ch += 2) copy16_async(Kb + ch * 8, ok ? ksrc + ch * 8 : cache, ok);
        const __nv_bfloat16* vsrc = page_base + v_base + (size_t)off * E + v0;
        for (int ch = fpar; ch < vchunks; ch += 2) {
            const bool in = ok && v0 + ch * 8 < E;
            copy16_async(Vb + ch * 8, in ? vsrc + ch * 8 : cache, in);
        }
        copies_commit();
    };
    // key tiles that no token of the tile sees are skipped: they would add exact zeros
    const int first_tile = first_visible(pos0, window, chunk) / BN;
    const int n_tiles = last_tile + 1 - first_tile, per = (n_tiles + nsplit - 1) / nsplit, kt_lo = first_tile + sp * per,
              kt_hi = min(last_tile + 1, kt_lo + per);
    if (kt_lo < kt_hi) fetch(kt_lo, 0);
    for (int kt = kt_lo; kt < kt_hi; ++kt) {
        const int j0 = kt * BN;
        if (kt + 1 < kt_hi) fetch(kt + 1, (kt + 1 - kt_lo) & 1);
        else copies_commit();
        copies_wait<1>();
        __syncthreads();                                                  // tile kt has landed for every thread
        const __nv_bfloat16* Kt = Ks + ((kt - kt_lo) & 1) * stage;
        const __nv_bfloat16* Vt = Vs + ((kt - kt_lo) & 1) * stage;

        // a warp whose 16 rows lie beyond the tile's rows (a single token brings H/G rows) has nothing to compute
        if (rb * 16 < rows) {
            // S = Q K^T for this warp's 16 rows and the tile's 64 keys
            float sacc[BN / 8][4];
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
            for (int k0 = 0; k0 < D; k0 += 16) {
                uint32_t a[4];
                ldmatrix_x4(a, Qs + (rb * 16 + (lane & 15)) * DP + k0 + (lane >> 4) * 8);
#pragma unroll
                for (int nt = 0; nt < BN / 8; nt += 2) {
                    uint32_t b[4];      // keys nt*8 .. nt*8+15: (b0, b1) of the first eight, (b0, b1) of the next eight
                    ldmatrix_x4(b, Kt + (nt * 8 + (lane & 7) + ((lane >> 4) << 3)) * DP + k0 + ((lane >> 3) & 1) * 8);
                    mma_bf16(sacc[nt], a, b[0], b[1]);
                    mma_bf16(sacc[nt + 1], a, b[2], b[3]);
                }
            }
            // scale, distance term, mask, and the tile's maximum per row.  A tile that every row of the CTA sees whole needs no mask.
            const bool whole = rows == BM && j0 + BN - 1 <= pos0 && j0 >= see_last;
            float tmax[2] = {-INFINITY, -INFINITY};
            if (whole && !r1 && softcap == 0.f) {
#pragma unroll
                for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        sacc[nt][e] *= sl2;
                        tmax[e >> 1] = fmaxf(tmax[e >> 1], sacc[nt][e]);
                    }
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = j0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        const int hi = e >> 1;
                        const int pos = hi ? pos_hi : pos_lo;
                        const bool ok = (hi ? live_hi : live_lo) && j <= pos && j >= (hi ? see_hi : see_lo);
                        float s = -INFINITY;
                        if (ok) {
                            s = softcap > 0.f ? cap_out * tanh_fast(sacc[nt][e] * cap_in) : sacc[nt][e] * sl2;
                            // r1 ln(1 + r2 d) in units of log2(e) is r1 log2(1 + r2 d); lg2.approx errs by 2^-22, far below
                            // the rounding of the bfloat16 operands of q . k
                            if (r1) s -= r1v[hi] * __log2f(fmaf(r2v[hi], (float)(pos - j), 1.0f));
                        }
                        sacc[nt][e] = s;
                        tmax[hi] = fmaxf(tmax[hi], s);
                    }
                }
            }
            float alpha[2], base[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
                const float m_new = fmaxf(row_m[h], tmax[h]);
                base[h] = m_new == -INFINITY ? 0.f : m_new;                   // a row that has seen nothing yet
                alpha[h] = ex2(row_m[h] - base[h]);                         // exp2(-inf) = 0
                row_m[h] = m_new;
            }
            float tsum[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) {                             // the weights stay in sacc, in fp32
                sacc[nt][0] = ex2(sacc[nt][0] - base[0]);
                sacc[nt][1] = ex2(sacc[nt][1] - base[0]);
                sacc[nt][2] = ex2(sacc[nt][2] - base[1]);
                sacc[nt][3] = ex2(sacc[nt][3] - base[1]);
                tsum[0] += sacc[nt][0] + sacc[nt][1];
                tsum[1] += sacc[nt][2] + sacc[nt][3];
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tsum[h] += __shfl_xor_sync(0xffffffffu, tsum[h], 1);
                tsum[h] += __shfl_xor_sync(0xffffffffu, tsum[h], 2);
                row_l[h] = row_l[h] * alpha[h] + tsum[h];
            }
#pragma unroll
            for (int i = 0; i < VC / 8; ++i) {
                if (i >= ntw) break;
                oacc[i][0] *= alpha[0];
                oacc[i][1] *= alpha[0];
                oacc[i][2] *= alpha[1];
                oacc[i][3] *= alpha[1];
            }
            // O += P V.  A weight enters the product as two bfloat16 numbers, its rounding and what the rounding left over
            // (16 bits of mantissa together): the weights are 32-bit numbers, and where the two maps' outputs nearly cancel a
            // weight rounded to 8 bits would show.
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
                uint32_t pa[4], pl[4];                                        // P as the A operand, 16 keys: rounded, and the rest
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const float* pv = sacc[2 * kk + half];
                    const __nv_bfloat162 h01 = __floats2bfloat162_rn(pv[0], pv[1]), h23 = __floats2bfloat162_rn(pv[2], pv[3]);
                    pa[half * 2] = *reinterpret_cast<const uint32_t*>(&h01);
                    pa[half * 2 + 1] = *reinterpret_cast<const uint32_t*>(&h23);
                    pl[half * 2] = pack_bf16(pv[0] - __low2float(h01), pv[1] - __high2float(h01));
                    pl[half * 2 + 1] = pack_bf16(pv[2] - __low2float(h23), pv[3] - __high2float(h23));
                }
#pragma unroll
                for (int nt = 0; nt < VC / 8; nt += 2) {
                    if (nt >= ntw) break;                                 // (the same for the whole warp)
                    uint32_t b[4];      // keys kk*16 .. +15 (rows), columns cb + nt*8 .. +15: matrices (k lo, n lo), (k hi, n lo), (k lo, n hi), (k hi, n hi)
                    ldmatrix_x4_trans(b, Vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VP + cb + nt * 8 + (lane >> 4) * 8);
                    mma_bf16(oacc[nt], pl, b[0], b[1]);
                    mma_bf16(oacc[nt + 1], pl, b[2], b[3]);
                    mma_bf16(oacc[nt], pa, b[0], b[1]);
                    mma_bf16(oacc[nt + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                                  // before a later fetch writes into this buffer
    }
    const float inv[2] = {nsplit > 1 ? 1.0f : (row_l[0] > 0.f ? 1.0f / row_l[0] : 0.f), nsplit > 1 ? 1.0f : (row_l[1] > 0.f ? 1.0f / row_l[1] : 0.f)};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = h ? r_hi : r_lo;
        if (r >= rows || rb * 16 >= rows) continue;
        const size_t head_index = (size_t)sp * T * H + (size_t)(t0 + r / Gq) * H + c * Gq + r % Gq;
        if (nsplit > 1 && blockIdx.z == 0 && (lane & 3) == 0 && (!colsplit || warp == 0)) {
            part_ml[(head_index * M + mp) * 2] = row_m[h];
            part_ml[(head_index * M + mp) * 2 + 1] = row_l[h];
        }
#pragma unroll
        for (int nt = 0; nt < VC / 8; ++nt) {
            if (nt >= ntw) break;
            const int col = v0 + cb + nt * 8 + (lane & 3) * 2;
            if (col >= E) continue;
            const float a = oacc[nt][2 * h] * inv[h], b = oacc[nt][2 * h + 1] * inv[h];
            if (M == 1 && nsplit == 1)
                *reinterpret_cast<uint32_t*>(out + (size_t)(t0 + r / Gq) * out_ld + (size_t)(c * Gq + r % Gq) * E + col) = pack_bf16(a * out_scale, b * out_scale);
            else *reinterpret_cast<float2*>(u + (head_index * M + mp) * E + col) = make_float2(a, b);
        }
    }
}

// A warp per (token, head): puts the runs of key tiles together (nsplit > 1: run s of a map counts with
// 2^(m_s - m) / sum_s 2^(m_s - m) l_s), and with two maps takes o = a_1 - lambda a_2 from u fp32 [nsplit, T, H, M, E], divides it
// by its root mean square (eps inside the root) and multiplies by post; with one map the output is the map's, times post.
// out bf16 [T, H, E].
__global__ void __launch_bounds__(128)
scored_combine_kernel(const float* __restrict__ u, const float* __restrict__ part_ml, int nsplit, __nv_bfloat16* __restrict__ out_base, int rows,
                      int H, int M, int E, float lambda, float post, float eps, long long out_ld) {
    constexpr int kMaxSplit = 16;
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= rows) return;
    __nv_bfloat16* orow = out_base + (size_t)(w / H) * out_ld + (size_t)(w % H) * E;      // where (token, head) w's values go
    float wt[2][kMaxSplit];              // the weight of run s of map m (not used with one run)
    for (int m = 0; m < M && nsplit > 1; ++m) {
        float mx = -INFINITY, den = 0.f;
        for (int s = 0; s < nsplit; ++s) mx = fmaxf(mx, part_ml[(((size_t)s * rows + w) * M + m) * 2]);
        for (int s = 0; s < nsplit; ++s) {
            const size_t at = (((size_t)s * rows + w) * M + m) * 2;
            const float l = part_ml[at + 1];
            const float x = l > 0.f ? exp2f(part_ml[at] - mx) : 0.f;          // a run that saw no key counts for nothing
            wt[m][s] = x;
            den = fmaf(x, l, den);
        }
        const float inv = den > 0.f ? 1.0f / den : 0.f;
        for (int s = 0; s < nsplit; ++s) wt[m][s] *= inv;
    }
    auto value = [&](int m, int e) {
        if (nsplit == 1) return u[((size_t)w * M + m) * E + e];
        float a = 0.f;
        for (int s = 0; s < nsplit; ++s) a = fmaf(wt[m][s], u[(((size_t)s * rows + w) * M + m) * E + e], a);
        return a;
    };
    if (M == 1) {
        for (int e = lane; e < E; e += 32) orow[e] = __float2bfloat16_rn(value(0, e) * post);
        return;
    }
    constexpr int kKeep = 8;             // heads of up to 256 values stay in registers between the two walks: u is read once
    float ss = 0.f, kept[kKeep];
    const bool keep = E <= 32 * kKeep;
    if (keep) {
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int e = lane + 32 * i;
            kept[i] = e < E ? value(0, e) - lambda * value(1, e) : 0.f;
            ss = fmaf(kept[i], kept[i], ss);
        }
    } else {
        for (int e = lane; e < E; e += 32) {
            const float o = value(0, e) - lambda * value(1, e);
            ss = fmaf(o, o, ss);
        }
    }
    ss = forge::warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)E + eps) * post;
    if (keep) {
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int e = lane + 32 * i;
            if (e < E) orow[e] = __float2bfloat16_rn(kept[i] * inv);
        }
    } else {
        for (int e = lane; e < E; e += 32) orow[e] = __float2bfloat16_rn((value(0, e) - lambda * value(1, e)) * inv);
    }
}

forge::PerDeviceFlag g_attr_done[6];

template <int VC, bool SPLIT>
int launch_scored(int which, dim3 grid, size_t smem, cudaStream_t stream, const __nv_bfloat16* q, const __nv_bfloat16* cache,
                  const int32_t* bt, const int32_t* tok_req, const int32_t* positions, const int32_t* t0, const int32_t* tn, const float* r1,
                  const float* r2, float* u, __nv_bfloat16* out, float* part_ml, int nsplit, int T, int qrows, int H, int G, int M, int D, int E,
                  int page_size, long long page_stride, int max_pages, float scale, float out_scale, long long out_ld, int window, int chunk,
                  float softcap) {
    bool& done = g_attr_done[which + (SPLIT ? 3 : 0)].current();
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(scored_mma_kernel<VC, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmemLimit);
        if (e != cudaSuccess) return forge::check_launch("scored_attention_mma (shared memory)", e);
        done = true;
    }
    return forge::check_launch("scored_attention_mma",
                               forge::launch(scored_mma_kernel<VC, SPLIT>, grid, dim3(kThreads), smem, stream, 1, q, cache, bt, tok_req, positions, t0,
                                             tn, r1, r2, u, out, part_ml, nsplit, T, qrows, H, G, M, D, E, page_size, page_stride, max_pages, scale,
                                             out_scale, out_ld, window, chunk, softcap));
}

}  // namespace

// 1 if the tensor-core kernel takes these sizes: maps of a multiple of 16 channels up to 128, value heads of a multiple of 8
// channels, at most 64 query heads per key/value head, pages of a power of two tokens.
extern "C" int forge_scored_mma_supports(int H, int G, int M, int D, int E, int page_size) {
    return (page_size > 0 && (page_size & (page_size - 1)) == 0 && H > 0 && G > 0 && H % G == 0 && H / G <= BM && (M == 1 || M == 2) &&
            D % 16 == 0 && D >= 16 && D <= 128 && E % 8 == 0 && E > 0) ? 1 : 0;
}

// q bf16 [T, H*M*D]; u fp32 [nsplit, T, H, M, E] (scratch; not needed with M == 1 and nsplit == 1); part_ml fp32
// [nsplit, T, H, M, 2] (scratch, nsplit > 1: steps of single tokens only); out bf16, rows of out_ld elements (even) with the
// heads' H*E values at their start.  tile_t0 / tile_n: tiles of consecutive
// tokens of one request with tile_n * (H/G) <= 64 (both null: one token per tile, num_tiles = T).  r1, r2 fp32 [H] or null.
// window, chunk, softcap: the limits on what a position sees and the cap on the scores, 0 = none.
extern "C" int forge_scored_attention_mma(const void* q, const void* cache, const int32_t* block_table, const int32_t* tok_req,
                                          const int32_t* positions, const int32_t* tile_t0, const int32_t* tile_n, const float* r1,
                                          const float* r2, float* u, float* part_ml, int nsplit, void* out, int T, int num_tiles, int H, int G, int M, int D, int E,
                                          int page_size, long long page_stride, int max_pages, float scale, float lambda, float post,
                                          float eps, float out_scale, long long out_ld, int window, int chunk, float softcap,
                                          cudaStream_t stream) {
    if (out_ld < (long long)H * E || (out_ld & 1)) return forge::fail(FORGE_ERR_ARG, "scored_attention_mma: output rows of %lld elements", out_ld);
    if (!forge_scored_mma_supports(H, G, M, D, E, page_size))
        return forge::fail(FORGE_ERR_UNSUPPORTED, "scored_attention_mma: H=%d G=%d M=%d D=%d E=%d", H, G, M, D, E);
    if (T < 0 || num_tiles < 0 || max_pages <= 0 || (tile_t0 == nullptr) != (tile_n == nullptr) || (r1 == nullptr) != (r2 == nullptr) ||
        ((M == 2 || nsplit > 1) && !u) || window < 0 || chunk < 0 || softcap < 0.f)
        return forge::fail(FORGE_ERR_ARG, "scored_attention_mma: bad arguments");
    if (nsplit < 1 || nsplit > 16 || (nsplit > 1 && (tile_t0 != nullptr || part_ml == nullptr)))
        return forge::fail(FORGE_ERR_ARG, "scored_attention_mma: the keys are dealt out to several CTAs only in steps of single tokens");
    if (T == 0 || num_tiles == 0) return FORGE_OK;
    int VC = 64;                        // the chunk width that wastes the fewest columns; among equals the widest
    for (int cand : {128, 256})
        if ((E + cand - 1) / cand * cand <= (E + VC - 1) / VC * VC) VC = cand;
    const int chunks = (E + VC - 1) / VC;
    // a step of single tokens brings H/G rows a tile: 16 rows of queries in shared memory leave room for more CTAs on the SM
    const int qrows = (tile_t0 == nullptr && H / G <= 16) ? 16 : BM;
    const size_t smem = sizeof(__nv_bfloat16) * ((size_t)qrows * (D + kPad) + 2 * (size_t)BN * ((D + kPad) + (VC + kPad)));
    const dim3 grid(num_tiles * nsplit, G * M, chunks);
    const __nv_bfloat16* qb = (const __nv_bfloat16*)q;
    const __nv_bfloat16* cb = (const __nv_bfloat16*)cache;
    __nv_bfloat16* ob = (__nv_bfloat16*)out;
    const float os = (M == 1 && nsplit == 1) ? out_scale : 1.0f;
    int rc;
#define FORGE_SCORED_ARGS grid, smem, stream, qb, cb, block_table, tok_req, positions, tile_t0, tile_n, r1, r2, u, ob, part_ml, nsplit, T, qrows, H, G, M, D, E, page_size, page_stride, max_pages, scale, os, out_ld, window, chunk, softcap
    if (nsplit > 1) rc = VC == 64 ? launch_scored<64, true>(0, FORGE_SCORED_ARGS) : VC == 128 ? launch_scored<128, true>(1, FORGE_SCORED_ARGS) : launch_scored<256, true>(2, FORGE_SCORED_ARGS);
    else rc = VC == 64 ? launch_scored<64, false>(0, FORGE_SCORED_ARGS) : VC == 128 ? launch_scored<128, false>(1, FORGE_SCORED_ARGS) : launch_scored<256, false>(2, FORGE_SCORED_ARGS);
#undef FORGE_SCORED_ARGS
    if (rc != FORGE_OK || (M == 1 && nsplit == 1)) return rc;
    const unsigned blocks = (unsigned)(((size_t)T * H + 3) / 4);
    return forge::check_launch("scored_combine", forge::launch(scored_combine_kernel, dim3(blocks), dim3(128), 0, stream, 1, (const float*)u,
                                                               (const float*)part_ml, nsplit, ob, T * H, H, M, E, lambda,
                                                               (M == 1 ? 1.0f : post) * out_scale, eps, out_ld));
}

FORGE_DEFINE_CHECKS_ENTRY(attention_scored_mma)
