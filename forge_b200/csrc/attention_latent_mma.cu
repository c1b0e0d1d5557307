// Tensor-core form (bf16 operands, fp32 sums) of the attention over latent rows, for prompt portions and single tokens
// alike; see attention_latent.cu for the definition and the cache layout (one row [c | kr] of C + R channels a token, the
// values are a row's first C channels, every head attends with an absorbed query of C + R channels over the same rows).
//
// A CTA of four warps takes a tile of up to 64 rows = consecutive tokens of one request x a group of up to 64 heads, one
// chunk of VC value columns, and walks the rows of the cache in tiles of 64 positions that start at multiples of 64: one
// tile in shared memory serves as keys (all C + R channels, the column-major operand of S = Q K^T) and as values (its
// columns of the chunk, through ldmatrix.trans, in O += P V).  Tiles go through two buffers where two fit beside the
// queries, else through one.  mma.sync m16n8k16 (the legacy tensor path).  Softmax in fp32 with a running maximum and sum
// per row in registers; a weight is the value product's operand as two bfloat16 numbers, its rounding and what the
// rounding left over (16 bits of mantissa).  A step of single tokens may deal a request's tiles out to several CTAs in
// runs; a second kernel puts the runs together.  Where the latent has an even number of value chunks, a prompt portion's CTA is
// eight warps: two sets of four over the same queries and tiles, each with a chunk of its own.
#include "common.cuh"
#include "checks.cuh"

namespace {

constexpr int BM = 64, BN = 64, kThreads = 128, kPad = 8;
constexpr int kSmemLimit = 200 * 1024;

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
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// q bf16 [T, H, KD] (KD = C + R), cache rows of KD.  nsplit == 1: out bf16 [T, H, C], normalised.  nsplit > 1 (steps of single
// tokens): run sp leaves its sums as they are in u fp32 [nsplit, T, H, C], beside the row's maximum (in units of log2 e) and
// sum in part_ml [nsplit, T, H, 2].
template <int VC, bool SPLIT>
__global__ void __launch_bounds__(2 * kThreads)
latent_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache, const int32_t* __restrict__ block_table,
                  const int32_t* __restrict__ tok_req, const int32_t* __restrict__ positions, const int32_t* __restrict__ tile_t0,
                  const int32_t* __restrict__ tile_n, float* __restrict__ u, __nv_bfloat16* __restrict__ out, float* __restrict__ part_ml,
                  int nsplit_given, int nbuf, int T, int qrows, int H, int HG, int C, int R, int page_size, int max_pages, float scale,
                  int window, const float* __restrict__ sink) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int nsplit = SPLIT ? nsplit_given : 1;
    // the last tiles of a prompt see the most keys: they start first, so that the short ones fill the grid's tail
    // A CTA of eight warps (prompt portions over a latent of an even number of value chunks) is two sets of four over the same
    // queries and tiles of rows, each set with a chunk of value columns of its own: twice the warps for the copies' latency to hide behind.
    const int nthreads = blockDim.x, halves = nthreads / kThreads;
    const int tile = gridDim.x / nsplit - 1 - blockIdx.x / nsplit, sp = blockIdx.x % nsplit;
    const int v0 = (blockIdx.z * halves + (int)(threadIdx.x / kThreads)) * VC;
    const int t0 = tile_t0 ? tile_t0[tile] : tile;
    const int nq = tile_n ? tile_n[tile] : 1;
    if (!FORGE_TOKEN_OK(t0) || !FORGE_TOKEN_OK(t0 + nq - 1)) return;
    const int h0 = blockIdx.y * HG, nh = min(HG, H - h0), rows = nq * nh, KD = C + R, KP = KD + kPad;
    const int pos0 = positions[t0], pos_last = pos0 + nq - 1;
    const int32_t* table = block_table + (size_t)tok_req[t0] * max_pages;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [qrows][KD + 8]
    __nv_bfloat16* Ks = Qs + qrows * KP;                                  // nbuf x [BN][KD + 8]
    const int stage = BN * KP;
    const int tid = threadIdx.x, lane = tid & 31, warp = (tid >> 5) & 3;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    // queries: row r = token t0 + r / nh, head h0 + r % nh
    const int dchunks = KD >> 3;
    for (int i = tid; i < qrows * dchunks; i += nthreads) {
        const int r = i / dchunks, ch = i % dchunks;
        uint4 val = zero4;
        if (r < rows) val = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + r / nh) * H + h0 + r % nh) * KD + ch * 8);
        *reinterpret_cast<uint4*>(Qs + r * KP + ch * 8) = val;
    }

    float oacc[VC / 8][4];
#pragma unroll
    for (int i = 0; i < VC / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
    float row_m[2] = {-INFINITY, -INFINITY}, row_l[2] = {0.f, 0.f};
    // A tile of at most 16 rows would leave three warps idle: there all four warps take the same 16 rows, each computes the
    // scores again, and each takes a quarter of the chunk's value columns.
    const int vcols = min(VC, C - v0);                                    // a multiple of 16
    const bool colsplit = rows <= 16 && vcols % 64 == 0;
    const int rb = colsplit ? 0 : warp;                                   // this warp's block of 16 rows
    const int ntw = colsplit ? vcols / 32 : vcols / 8, cb = colsplit ? warp * (vcols / 4) : 0;     // its value columns: ntw blocks of 8 from cb
    const int r_lo = rb * 16 + (lane >> 2), r_hi = r_lo + 8;             // this thread's two rows
    const int pos_lo = pos0 + min(r_lo, rows - 1) / nh, pos_hi = pos0 + min(r_hi, rows - 1) / nh;
    const bool live_lo = r_lo < rows, live_hi = r_hi < rows;
    // the first row each of the thread's two positions sees, and the tile's last token (no token of the tile sees an earlier row)
    const int see_lo = window > 0 ? max(0, pos_lo - window + 1) : 0, see_hi = window > 0 ? max(0, pos_hi - window + 1) : 0;
    const int see_last = window > 0 ? max(0, pos_last - window + 1) : 0;

    const int last_tile = pos_last / BN;
    constexpr float kLog2e = 1.4426950408889634f;
    const float sl2 = scale * kLog2e;                                     // scores in units of log2(e)
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;

    const int per_row = nthreads / BN, frow = tid / per_row, fpar = tid % per_row;   // two (or four) threads a cache row
    auto fetch = [&](int kt, int buf) {
        const int j = kt * BN + frow;
        __nv_bfloat16* Kb = Ks + buf * stage + frow * KP;
        const __nv_bfloat16* src = cache;
        bool ok = false;
        if (j <= pos_last) {
            const int page = table[j >> page_shift];
            if (page >= 0 && FORGE_PAGE_OK(page)) {
                ok = true;
                src = cache + ((size_t)page * page_size + (j & (page_size - 1))) * KD;
            }
        }
        for (int ch = fpar; ch < dchunks; ch += per_row) copy16_async(Kb + ch * 8, ok ? src + ch * 8 : cache, ok);
        copies_commit();
    };
    // tiles of rows behind every token's window are skipped: they would add exact zeros
    const int first_tile = (window > 0 ? max(0, pos0 - window + 1) : 0) / BN;
    const int n_tiles = last_tile + 1 - first_tile, per = (n_tiles + nsplit - 1) / nsplit, kt_lo = first_tile + sp * per,
              kt_hi = min(last_tile + 1, kt_lo + per);
    if (kt_lo < kt_hi) fetch(kt_lo, 0);
    for (int kt = kt_lo; kt < kt_hi; ++kt) {
        const int j0 = kt * BN;
        const int buf = nbuf == 2 ? ((kt - kt_lo) & 1) : 0;
        if (nbuf == 2 && kt + 1 < kt_hi) fetch(kt + 1, buf ^ 1);
        else copies_commit();
        copies_wait<1>();
        __syncthreads();                                                  // tile kt has landed for every thread
        const __nv_bfloat16* Kt = Ks + buf * stage;

        // a warp whose 16 rows lie beyond the tile's rows has nothing to compute
        if (rb * 16 < rows) {
            float sacc[BN / 8][4];
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
            for (int k0 = 0; k0 < KD; k0 += 16) {
                uint32_t a[4];
                ldmatrix_x4(a, Qs + (rb * 16 + (lane & 15)) * KP + k0 + (lane >> 4) * 8);
#pragma unroll
                for (int nt = 0; nt < BN / 8; nt += 2) {
                    uint32_t b[4];      // keys nt*8 .. nt*8+15: (b0, b1) of the first eight, (b0, b1) of the next eight
                    ldmatrix_x4(b, Kt + (nt * 8 + (lane & 7) + ((lane >> 4) << 3)) * KP + k0 + ((lane >> 3) & 1) * 8);
                    mma_bf16(sacc[nt], a, b[0], b[1]);
                    mma_bf16(sacc[nt + 1], a, b[2], b[3]);
                }
            }
            // scale, mask, and the tile's maximum per row.  A tile that every row of the CTA sees whole needs no mask.
            const bool whole = rows == qrows && qrows == BM && j0 + BN - 1 <= pos0 && j0 >= see_last;
            float tmax[2] = {-INFINITY, -INFINITY};
            if (whole) {
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
                        const bool ok = (hi ? live_hi : live_lo) && j <= (hi ? pos_hi : pos_lo) && j >= (hi ? see_hi : see_lo);
                        const float s = ok ? sacc[nt][e] * sl2 : -INFINITY;
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
            // O += P V, the values being the tile's own columns v0 + cb ...
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
                    uint32_t b[4];      // keys kk*16 .. +15 (rows), columns .. +15: matrices (k lo, n lo), (k hi, n lo), (k lo, n hi), (k hi, n hi)
                    ldmatrix_x4_trans(b, Kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KP + v0 + cb + nt * 8 + (lane >> 4) * 8);
                    mma_bf16(oacc[nt], pl, b[0], b[1]);
                    mma_bf16(oacc[nt + 1], pl, b[2], b[3]);
                    mma_bf16(oacc[nt], pa, b[0], b[1]);
                    mma_bf16(oacc[nt + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();                                                  // before a later fetch writes into this buffer
        if (nbuf == 1 && kt + 1 < kt_hi) fetch(kt + 1, 0);
    }
    if (sink != nullptr && nsplit == 1) {
        // a sink joins the denominator as one more weight, exp(sink_h), that has no row of its own (maxima are in units of log2 e)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = min(h ? r_hi : r_lo, rows - 1);
            if (row_l[h] > 0.f) row_l[h] += ex2(sink[h0 + r % nh] * kLog2e - row_m[h]);
        }
    }
    const float inv[2] = {nsplit > 1 ? 1.0f : (row_l[0] > 0.f ? 1.0f / row_l[0] : 0.f), nsplit > 1 ? 1.0f : (row_l[1] > 0.f ? 1.0f / row_l[1] : 0.f)};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = h ? r_hi : r_lo;
        if (r >= rows || rb * 16 >= rows) continue;
        const size_t head_index = (size_t)sp * T * H + (size_t)(t0 + r / nh) * H + h0 + r % nh;
        if (nsplit > 1 && v0 == 0 && (lane & 3) == 0 && (!colsplit || warp == 0)) {
            part_ml[head_index * 2] = row_m[h];
            part_ml[head_index * 2 + 1] = row_l[h];
        }
#pragma unroll
        for (int nt = 0; nt < VC / 8; ++nt) {
            if (nt >= ntw) break;
            const int col = v0 + cb + nt * 8 + (lane & 3) * 2;
            const float a = oacc[nt][2 * h] * inv[h], b = oacc[nt][2 * h + 1] * inv[h];
            if (nsplit == 1) *reinterpret_cast<uint32_t*>(out + head_index * C + col) = pack_bf16(a, b);
            else *reinterpret_cast<float2*>(u + head_index * C + col) = make_float2(a, b);
        }
    }
}

// A warp per (token, head): run s counts with 2^(m_s - m); the sums of all runs over the sum of their weights' sums.
__global__ void __launch_bounds__(128)
latent_combine_kernel(const float* __restrict__ u, const float* __restrict__ part_ml, int nsplit, __nv_bfloat16* __restrict__ out, int rows, int C,
                      const float* __restrict__ sink, int H) {
    constexpr int kMaxSplit = 16;
    forge::pdl_launch_dependents();
    forge::pdl_wait();
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= rows) return;
    float wt[kMaxSplit];
    float m = -INFINITY;
    for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[((size_t)s * rows + w) * 2]);
    float l = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxSplit; ++s) {
        wt[s] = 0.f;
        if (s < nsplit) {
            const float ms = part_ml[((size_t)s * rows + w) * 2];
            wt[s] = ms == -INFINITY ? 0.f : ex2(ms - m);
            l += wt[s] * part_ml[((size_t)s * rows + w) * 2 + 1];
        }
    }
    if (sink != nullptr && l > 0.f) l += ex2(sink[w % H] * 1.4426950408889634f - m);      // the sink's weight in the denominator
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    // four channels a load (C is a multiple of 16), all runs' loads of a channel group in flight together
    for (int c = lane * 4; c < C; c += 128) {
        float4 part[kMaxSplit];
#pragma unroll
        for (int s = 0; s < kMaxSplit; ++s)
            if (s < nsplit && wt[s] != 0.f) part[s] = *reinterpret_cast<const float4*>(u + ((size_t)s * rows + w) * C + c);
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < kMaxSplit; ++s)
            if (s < nsplit && wt[s] != 0.f) {
                a.x = fmaf(wt[s], part[s].x, a.x); a.y = fmaf(wt[s], part[s].y, a.y);
                a.z = fmaf(wt[s], part[s].z, a.z); a.w = fmaf(wt[s], part[s].w, a.w);
            }
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(out + (size_t)w * C + c);
        o[0] = __floats2bfloat162_rn(a.x * inv, a.y * inv);
        o[1] = __floats2bfloat162_rn(a.z * inv, a.w * inv);
    }
}

forge::PerDeviceFlag g_attr_done[6];

template <int VC, bool SPLIT>
int launch_latent(int which, dim3 grid, size_t smem, cudaStream_t stream, const __nv_bfloat16* q, const __nv_bfloat16* cache, const int32_t* bt,
                  const int32_t* tok_req, const int32_t* positions, const int32_t* t0, const int32_t* tn, float* u, __nv_bfloat16* out,
                  float* part_ml, int nsplit, int nbuf, int T, int qrows, int H, int HG, int C, int R, int page_size, int max_pages, float scale, int halves,
                  int window, const float* sink) {
    bool& done = g_attr_done[which + (SPLIT ? 3 : 0)].current();
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(latent_mma_kernel<VC, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
        if (e != cudaSuccess) return forge::check_launch("latent_attention_mma (shared memory)", e);
        done = true;
    }
    return forge::check_launch("latent_attention_mma",
                               forge::launch(latent_mma_kernel<VC, SPLIT>, grid, dim3(kThreads * halves), smem, stream, 1, q, cache, bt, tok_req, positions, t0,
                                             tn, u, out, part_ml, nsplit, nbuf, T, qrows, H, HG, C, R, page_size, max_pages, scale, window, sink));
}

size_t latent_mma_smem(int qrows, int KD, int nbuf) { return sizeof(__nv_bfloat16) * (size_t)(qrows + nbuf * BN) * (KD + kPad); }

}  // namespace

// 1 if the tensor-core kernel takes these sizes: a latent and a rotated part of a multiple of 16 channels each, rows that fit
// shared memory beside a tile of queries, pages of a power of two tokens.
extern "C" int forge_latent_mma_supports(int H, int C, int R, int page_size) {
    return (page_size > 0 && (page_size & (page_size - 1)) == 0 && H > 0 && C >= 16 && C % 16 == 0 && R >= 0 && R % 16 == 0 &&
            latent_mma_smem(BM, C + R, 1) <= (size_t)kSmemLimit) ? 1 : 0;
}

// Heads a CTA takes (the caller cuts the step into tiles of 64 / this many tokens).
extern "C" int forge_latent_mma_heads(int H) { return H < BM ? H : BM; }

// q bf16 [T, H*(C+R)]; out bf16 [T, H*C]; u fp32 [nsplit, T, H, C] and part_ml fp32 [nsplit, T, H, 2] (scratch, nsplit > 1: steps of
// single tokens only).  tile_t0 / tile_n: tiles of consecutive tokens of one request with tile_n * min(H, 64) <= 64 (both null:
// one token per tile, num_tiles = T).  window: position i reads the rows j with i - window < j <= i (0: every j <= i);
// sink fp32 [H] or null: exp(sink_h) is added to head h's softmax denominator.
extern "C" int forge_latent_attention_mma(const void* q, const void* cache, const int32_t* block_table, const int32_t* tok_req,
                                          const int32_t* positions, const int32_t* tile_t0, const int32_t* tile_n, float* u, float* part_ml,
                                          int nsplit, void* out, int T, int num_tiles, int H, int C, int R, int page_size, int max_pages,
                                          float scale, int window, const float* sink, cudaStream_t stream) {
    if (!forge_latent_mma_supports(H, C, R, page_size)) return forge::fail(FORGE_ERR_UNSUPPORTED, "latent_attention_mma: H=%d C=%d R=%d", H, C, R);
    if (T < 0 || num_tiles < 0 || max_pages <= 0 || (tile_t0 == nullptr) != (tile_n == nullptr))
        return forge::fail(FORGE_ERR_ARG, "latent_attention_mma: bad arguments");
    if (nsplit < 1 || nsplit > 16 || (nsplit > 1 && (tile_t0 != nullptr || part_ml == nullptr || u == nullptr)))
        return forge::fail(FORGE_ERR_ARG, "latent_attention_mma: the rows are dealt out to several CTAs only in steps of single tokens");
    if (T == 0 || num_tiles == 0) return FORGE_OK;
    int VC = 64;                        // the chunk width that wastes the fewest columns; among equals the widest
    for (int cand : {128, 256})
        if ((C + cand - 1) / cand * cand <= (C + VC - 1) / VC * VC) VC = cand;
    const int chunks = (C + VC - 1) / VC, HG = forge_latent_mma_heads(H), KD = C + R;
    // a step of single tokens brings at most HG rows a tile: 16 rows of queries in shared memory leave room for more CTAs on the SM
    const int qrows = (tile_t0 == nullptr && HG <= 16) ? 16 : BM;
    const int nbuf = latent_mma_smem(qrows, KD, 2) <= (size_t)kSmemLimit ? 2 : 1;
    const size_t smem = latent_mma_smem(qrows, KD, nbuf);
    // prompt portions over a latent of an even number of value chunks: a CTA of eight warps takes two chunks (a step of single
    // tokens has at most two warps' worth of rows a tile and measured slower that way: 84 -> 93 us at 64 requests)
    const int halves = (tile_t0 != nullptr && nsplit == 1 && chunks % 2 == 0) ? 2 : 1;
    const dim3 grid(num_tiles * nsplit, (H + HG - 1) / HG, chunks / halves);
    const __nv_bfloat16* qb = (const __nv_bfloat16*)q;
    const __nv_bfloat16* cb = (const __nv_bfloat16*)cache;
    __nv_bfloat16* ob = (__nv_bfloat16*)out;
    int rc;
#define FORGE_LATENT_ARGS grid, smem, stream, qb, cb, block_table, tok_req, positions, tile_t0, tile_n, u, ob, part_ml, nsplit, nbuf, T, qrows, H, HG, C, R, page_size, max_pages, scale, halves, window, sink
    if (nsplit > 1) rc = VC == 64 ? launch_latent<64, true>(0, FORGE_LATENT_ARGS) : VC == 128 ? launch_latent<128, true>(1, FORGE_LATENT_ARGS) : launch_latent<256, true>(2, FORGE_LATENT_ARGS);
    else rc = VC == 64 ? launch_latent<64, false>(0, FORGE_LATENT_ARGS) : VC == 128 ? launch_latent<128, false>(1, FORGE_LATENT_ARGS) : launch_latent<256, false>(2, FORGE_LATENT_ARGS);
#undef FORGE_LATENT_ARGS
    if (rc != FORGE_OK || nsplit == 1) return rc;
    const unsigned blocks = (unsigned)(((size_t)T * H + 3) / 4);
    return forge::check_launch("latent_combine", forge::launch(latent_combine_kernel, dim3(blocks), dim3(128), 0, stream, 1, (const float*)u,
                                                               (const float*)part_ml, nsplit, ob, T * H, C, sink, H));
}

FORGE_DEFINE_CHECKS_ENTRY(attention_latent_mma)
