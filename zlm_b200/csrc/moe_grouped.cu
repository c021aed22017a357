// Routed experts for steps of many tokens (bf16): the (token, choice) pairs are sorted by expert on the
// device, and each expert's rows go through its two matrices as tiles of one grouped product on the
// warp-level tensor cores (mma.sync m16n8k16 behind a 4-stage cp.async pipeline), so that an expert's
// weights are read once per tile of rows instead of once per token.  Nothing comes back to the host:
// the tile table (which expert, which rows) is written by the sort kernel and read by the products,
// whose grids are sized for the most tiles the step can have.
//   moe_sort         pairs -> perm (sorted place -> pair), inv (pair -> sorted place), the tile table
//   grouped up       a[i, :] = act(w_i * (W_up[e] x[token(i)])) for the sorted rows i of expert e
//                    (rows of x gathered through perm; act = relu^2, the weight on the input side)
//   grouped down     y[i, :] = W_down[e] a[i, :]   (fp32)
//   moe_combine      stream[t, :] += sum_j y[inv[t, j], :], choices in their order
#include "common.cuh"
#include "attn_common.cuh"

#define MG_BK 32
#define MG_LD (MG_BK + 8)
#define MG_STAGES 4
#define MG_THREADS 256

__device__ __forceinline__ void mg_cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = (valid && ZLM_CHK(gmem, 16)) ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}

// ---------------------------------------------------------------------------- sort
// One block.  counts and cursors in shared memory (E entries each); tile table: tile -> (expert, first
// sorted row, rows), expert -1 for the tiles a step does not need.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ idx, int P, int E, int BM, int max_tiles, int padded, int drop, int* __restrict__ perm,
                int* __restrict__ inv, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                int* __restrict__ tile_rows) {
    extern __shared__ int sh[];
    int* count = sh;              // [E]
    int* start = sh + E;          // [E + 1] first sorted row of each expert
    int* tstart = start + E + 1;  // [E + 1] first tile of each expert
    pdl_trigger();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    pdl_wait();
    // padded: every expert's rows start at a tile's first row, and the rows between are marked empty
    if (padded)
        for (int i = threadIdx.x; i < max_tiles * BM; i += blockDim.x)
            if (ZLM_CHK(perm + i, 4)) perm[i] = -1;
    __syncthreads();
    // drop: a pair whose index is E or more (an expert without matrices) gets no row; its inv is -1
    for (int i = threadIdx.x; i < P; i += blockDim.x)
        if (ZLM_CHK(idx + i, 4) && !(drop && idx[i] >= E)) atomicAdd(&count[min(max(idx[i], 0), E - 1)], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0, t = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = padded ? t * BM : s;
            tstart[e] = t;
            s += count[e];
            t += (count[e] + BM - 1) / BM;
        }
        start[E] = padded ? t * BM : s;
        tstart[E] = t;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int n = count[e];
        for (int j = 0, t = tstart[e]; j * BM < n; ++j, ++t)
            if (t < max_tiles && ZLM_CHK(tile_expert + t, 4) && ZLM_CHK(tile_row0 + t, 4) && ZLM_CHK(tile_rows + t, 4)) {
                tile_expert[t] = e;
                tile_row0[t] = start[e] + j * BM;
                tile_rows[t] = min(BM, n - j * BM);
            }
        count[e] = 0;            // from here on: the expert's cursor
    }
    for (int t = tstart[E] + threadIdx.x; t < max_tiles; t += blockDim.x)
        if (ZLM_CHK(tile_expert + t, 4)) tile_expert[t] = -1;
    __syncthreads();
    // a pair's place among its expert's rows is whatever the cursor gives it: a row's result does not depend
    // on its place, and the combine step finds it through inv
    // (lanes that hold the same expert adding once through their first lane was measured: twice as slow)
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
        if (!ZLM_CHK(idx + i, 4)) continue;
        if (drop && idx[i] >= E) {
            if (ZLM_CHK(inv + i, 4)) inv[i] = -1;
            continue;
        }
        const int e = min(max(idx[i], 0), E - 1);
        const int place = start[e] + atomicAdd(&count[e], 1);
        if (ZLM_CHK(perm + place, 4) && ZLM_CHK(inv + i, 4)) {
            perm[place] = i;
            inv[i] = place;
        }
    }
}

// ---------------------------------------------------------------------------- grouped products
__device__ __forceinline__ float mg_relu2(float z) { z = fmaxf(z, 0.f); return z * z; }

// MODE 0 (up): rows of X gathered by perm, Y bf16 [sorted row, N] = act with the pair's weight
// MODE 1 (down): A = sorted rows [.., K], Y fp32 [sorted row, N]
// MODE 2 (per-head products of many tokens): group = head blockIdx.z, rows = tokens; A[t, head] and Y[t, head]
//         (bf16) lie a_hs and y_hs elements apart inside a token's row
template <int BM, int BN, int WARPS_M, int WARPS_N, int MODE>
__global__ void __launch_bounds__(MG_THREADS)
moe_grouped_kernel(void* __restrict__ Y, const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W,
                   const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                   const int* __restrict__ tile_rows, const int* __restrict__ perm, const float* __restrict__ wgt,
                   int top, int N, int K, int lda, int ldy, int scale_input, int T, int a_hs, int y_hs) {
    constexpr int WM = BM / WARPS_M, WN = BN / WARPS_N;
    constexpr int MT = WM / 16, NT = WN / 8;
    static_assert(WARPS_M * WARPS_N == MG_THREADS / 32 && WM % 16 == 0 && WN % 16 == 0, "warp tiles");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* As = (__nv_bfloat16*)smem_raw;                      // [STAGES][BM][LD]
    __nv_bfloat16* Bs = As + (size_t)MG_STAGES * BM * MG_LD;           // [STAGES][BN][LD]
    __shared__ const __nv_bfloat16* arow[BM];
    __shared__ float roww[BM];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp / WARPS_N, wn = warp % WARPS_N;
    pdl_launch_dependents();
    pdl_wait();
    int e, row0, rows;
    if (MODE == 2) {
        e = blockIdx.z;
        row0 = blockIdx.y * BM;
        rows = min(BM, T - row0);
    } else {
        if (!ZLM_CHK(tile_expert + blockIdx.y, 4)) return;
        e = tile_expert[blockIdx.y];
        if (e < 0) return;
        row0 = tile_row0[blockIdx.y];
        rows = tile_rows[blockIdx.y];
    }
    const int n0 = blockIdx.x * BN;
    const __nv_bfloat16* We = W + (size_t)e * N * K;
    for (int r = tid; r < BM; r += MG_THREADS) {
        const __nv_bfloat16* p = nullptr;
        float w = 0.f;
        if (MODE == 2) {
            if (r < rows) p = A + (size_t)(row0 + r) * lda + (size_t)e * a_hs;
        } else if (r < rows && ZLM_CHK(perm + row0 + r, 4)) {
            const int pair = perm[row0 + r];
            p = MODE == 0 ? A + (size_t)(pair / top) * lda : A + (size_t)(row0 + r) * lda;
            if (MODE == 0 && ZLM_CHK(wgt + pair, 4)) w = wgt[pair];
        }
        arow[r] = p;
        roww[r] = w;
    }
    __syncthreads();
    const int KT = (K + MG_BK - 1) / MG_BK;

    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.f;

    auto load_tile = [&](int kt, int stage) {
        const int k0 = kt * MG_BK;
        __nv_bfloat16* a = As + (size_t)stage * BM * MG_LD;
        __nv_bfloat16* b = Bs + (size_t)stage * BN * MG_LD;
        for (int id = tid; id < BM * 4; id += MG_THREADS) {
            const int r = id >> 2, c = (id & 3) * 8;
            const bool ok = arow[r] != nullptr && k0 + c < K;
            mg_cp_async16(a + r * MG_LD + c, ok ? arow[r] + k0 + c : A, ok);
        }
        for (int id = tid; id < BN * 4; id += MG_THREADS) {
            const int r = id >> 2, c = (id & 3) * 8;
            const bool ok = n0 + r < N && k0 + c < K;
            mg_cp_async16(b + r * MG_LD + c, ok ? We + (size_t)(n0 + r) * K + k0 + c : W, ok);
        }
    };
#pragma unroll
    for (int s = 0; s < MG_STAGES - 1; ++s) {
        if (s < KT) load_tile(s, s);
        dec_commit();
    }
    for (int kt = 0; kt < KT; ++kt) {
        dec_wait<MG_STAGES - 2>();
        __syncthreads();
        const int nk = kt + MG_STAGES - 1;
        if (nk < KT) load_tile(nk, nk % MG_STAGES);
        dec_commit();
        const __nv_bfloat16* a = As + (size_t)(kt % MG_STAGES) * BM * MG_LD;
        const __nv_bfloat16* b = Bs + (size_t)(kt % MG_STAGES) * BN * MG_LD;
#pragma unroll
        for (int ks = 0; ks < MG_BK; ks += 16) {
            unsigned af[MT][4], bf[NT][2];
#pragma unroll
            for (int i = 0; i < MT; ++i)
                dec_ldsm4(af[i][0], af[i][1], af[i][2], af[i][3],
                          a + (wm * WM + i * 16 + (lane & 15)) * MG_LD + ks + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
                const int mi = lane >> 3;
                dec_ldsm4(bf[j][0], bf[j][1], bf[j + 1][0], bf[j + 1][1],
                          b + (wn * WN + j * 8 + (mi >> 1) * 8 + (lane & 7)) * MG_LD + ks + (mi & 1) * 8);
            }
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) dec_mma(acc[i][j], af[i], bf[j][0], bf[j][1]);
        }
    }
    dec_wait<0>();

    const int g = lane >> 2, q = lane & 3;
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = wm * WM + i * 16 + g + half * 8;
            if (r >= rows) continue;
            const size_t orow = (size_t)(row0 + r) * ldy + (MODE == 2 ? (size_t)e * y_hs : 0);
            const float w = roww[r];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int n = n0 + wn * WN + j * 8 + q * 2;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    if (n + c >= N) continue;
                    const float v = acc[i][j][half * 2 + c];
                    if (MODE == 0) {
                        if (ZLM_CHK((__nv_bfloat16*)Y + orow + n + c, 2))
                            ((__nv_bfloat16*)Y)[orow + n + c] =
                                __float2bfloat16_rn(scale_input ? mg_relu2(w * v) : w * mg_relu2(v));
                    } else if (MODE == 2) {
                        if (ZLM_CHK((__nv_bfloat16*)Y + orow + n + c, 2)) ((__nv_bfloat16*)Y)[orow + n + c] = __float2bfloat16_rn(v);
                    } else if (ZLM_CHK((float*)Y + orow + n + c, 4)) {
                        ((float*)Y)[orow + n + c] = v;
                    }
                }
            }
        }
}

// stream[t, :] += sum_j y[inv[t * top + j], :]; one block per token
__global__ void __launch_bounds__(256)
moe_combine_kernel(float* __restrict__ stream, const float* __restrict__ y, const int* __restrict__ inv,
                   const float* __restrict__ wgt, int top, int N, const __nv_bfloat16* __restrict__ x = nullptr, int x_stride = 0,
                   const float* __restrict__ xw = nullptr) {
    // a pair without a row (inv < 0: an identity expert) adds xw * x[t] instead, if x is given
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (N % 4 == 0 && ((uintptr_t)y % 16 == 0) && ((uintptr_t)stream % 16 == 0)) {
        // four columns a thread; a column's sum runs over the choices in their order either way
        for (int n = threadIdx.x * 4; n < N; n += blockDim.x * 4) {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < top; ++j) {
                if (!ZLM_CHK(inv + (size_t)t * top + j, 4)) continue;
                if (inv[(size_t)t * top + j] < 0) {
                    const __nv_bfloat16* xr = x + (size_t)t * x_stride + n;
                    if (!x || !ZLM_CHK(xr, 8) || !ZLM_CHK(xw + (size_t)t * top + j, 4)) continue;
                    const float w = xw[(size_t)t * top + j];
                    sum.x += w * __bfloat162float(xr[0]); sum.y += w * __bfloat162float(xr[1]);
                    sum.z += w * __bfloat162float(xr[2]); sum.w += w * __bfloat162float(xr[3]);
                    continue;
                }
                const float* row = y + (size_t)inv[(size_t)t * top + j] * N + n;
                if (!ZLM_CHK(row, 16)) continue;
                const float4 v = *(const float4*)row;
                const float w = wgt ? wgt[(size_t)t * top + j] : 1.0f;
                sum.x += v.x * w; sum.y += v.y * w; sum.z += v.z * w; sum.w += v.w * w;
            }
            float* dst = stream + (size_t)t * N + n;
            if (!ZLM_CHK(dst, 16)) continue;
            float4 o = *(float4*)dst;
            o.x += sum.x; o.y += sum.y; o.z += sum.z; o.w += sum.w;
            *(float4*)dst = o;
        }
        return;
    }
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
        float sum = 0.f;
        for (int j = 0; j < top; ++j) {
            if (!ZLM_CHK(inv + (size_t)t * top + j, 4)) continue;
            if (inv[(size_t)t * top + j] < 0) {
                if (x && ZLM_CHK(x + (size_t)t * x_stride + n, 2) && ZLM_CHK(xw + (size_t)t * top + j, 4))
                    sum += xw[(size_t)t * top + j] * __bfloat162float(x[(size_t)t * x_stride + n]);
                continue;
            }
            if (ZLM_CHK(y + (size_t)inv[(size_t)t * top + j] * N + n, 4))
                sum += y[(size_t)inv[(size_t)t * top + j] * N + n] * (wgt ? wgt[(size_t)t * top + j] : 1.0f);
        }
        if (ZLM_CHK(stream + (size_t)t * N + n, 4)) stream[(size_t)t * N + n] += sum;
    }
}

// rows of a tile for P pairs over E experts: small tiles while an expert gets few rows
extern "C" int zlm_moe_grouped_tile_rows(int P, int E) {
    const int per = (P + E - 1) / E;
    return per <= 24 ? 16 : (per <= 192 ? 64 : 128);
}
// the most tiles a step of P pairs can need
extern "C" int zlm_moe_grouped_max_tiles(int P, int E, int BM) { return (P + BM - 1) / BM + (E < P ? E : P); }

template <int BM, int BN, int WARPS_M, int WARPS_N, int MODE>
static int launch_grouped(void* Y, const void* A, const void* W, const int* tiles, int max_tiles, const int* perm,
                          const float* wgt, int top, int N, int K, int lda, int ldy, int scale_input, cudaStream_t st) {
    const size_t smem = (size_t)MG_STAGES * (BM + BN) * MG_LD * sizeof(__nv_bfloat16);
    auto kern = moe_grouped_kernel<BM, BN, WARPS_M, WARPS_N, MODE>;
    static bool attr_set_dev[64] = {};
    bool& attr_set = attr_set_dev[zlm_device_index()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            zlm_set_error("moe_grouped: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return ZLM_ERR_CUDA;
        }
        attr_set = true;
    }
    dim3 grid((N + BN - 1) / BN, max_tiles);
    zlm_launch(kern, grid, dim3(MG_THREADS), smem, st, Y, (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, tiles,
               tiles + max_tiles, tiles + 2 * max_tiles, perm, wgt, top, N, K, lda, ldy, scale_input, 0, 0, 0);
    return zlm_check_launch("moe_grouped");
}

// out[t, h, :N] = W[h] x[t, h, :K] for many tokens (bf16): one product per head, tiles of tokens on the tensor cores
template <int BM>
static int launch_heads(void* out, int out_stride, int out_hs, const void* x, int x_stride, int x_hs, const void* W, int T,
                        int H, int N, int K, cudaStream_t st) {
    const size_t smem = (size_t)MG_STAGES * (BM + 128) * MG_LD * sizeof(__nv_bfloat16);
    auto kern = moe_grouped_kernel<BM, 128, 2, 4, 2>;
    static bool attr_set_dev[64] = {};
    bool& attr_set = attr_set_dev[zlm_device_index()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            zlm_set_error("head_linear_mma: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            return ZLM_ERR_CUDA;
        }
        attr_set = true;
    }
    dim3 grid((N + 127) / 128, (T + BM - 1) / BM, H);
    zlm_launch(kern, grid, dim3(MG_THREADS), smem, st, out, (const __nv_bfloat16*)x, (const __nv_bfloat16*)W,
               (const int*)nullptr, (const int*)nullptr, (const int*)nullptr, (const int*)nullptr, (const float*)nullptr, 1,
               N, K, x_stride, out_stride, 0, T, x_hs, out_hs);
    return zlm_check_launch("head_linear_mma");
}

extern "C" int zlm_head_linear_mma_supported(int K, int x_stride, int x_hs) {
    return (K % 8 == 0 && x_stride % 8 == 0 && x_hs % 8 == 0) ? 1 : 0;
}

extern "C" int zlm_head_linear_mma(void* out, int out_stride, int out_hs, const void* x, int x_stride, int x_hs,
                                   const void* W, int T, int H, int N, int K, cudaStream_t st) {
    if (T == 0 || N == 0) return ZLM_OK;
    ZLM_REQUIRE(T > 0 && H > 0 && H <= 65535 && N > 0 && K > 0, "head_linear_mma: bad sizes T=%d heads=%d N=%d K=%d", T, H, N, K);
    ZLM_REQUIRE(zlm_head_linear_mma_supported(K, x_stride, x_hs) && (uintptr_t)x % 16 == 0 && (uintptr_t)W % 16 == 0,
                "head_linear_mma: K=%d and the strides of x must be multiples of 8, operands 16-byte aligned", K);
    ZLM_REQUIRE((T + 63) / 64 <= 65535, "head_linear_mma: too many tokens (%d)", T);
    if (T > 64) return launch_heads<128>(out, out_stride, out_hs, x, x_stride, x_hs, W, T, H, N, K, st);
    return launch_heads<64>(out, out_stride, out_hs, x, x_stride, x_hs, W, T, H, N, K, st);
}

// The experts of a step of T tokens, `top` choices each (idx, wgt [T, top]): stream += sum of the chosen
// experts' outputs.  Scratch (the caller's): ints [2 * P + 3 * max_tiles], act bf16 [P, F], y fp32 [P, N], with
// P = T * top and max_tiles = zlm_moe_grouped_max_tiles(P, E, zlm_moe_grouped_tile_rows(P, E)).
extern "C" int zlm_moe_grouped(float* stream, const void* x, int x_stride, const void* Wup, const void* Wdown,
                               const int* idx, const float* wgt, int T, int top, int E, int F, int K,
                               int scale_input, int* ints, void* act, float* y, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    const int P = T * top;
    ZLM_REQUIRE(E > 0 && E <= 2048 && top > 0 && F > 0 && K > 0, "moe_grouped: experts=%d top=%d F=%d K=%d", E, top, F, K);
    ZLM_REQUIRE(K % 8 == 0 && F % 8 == 0 && x_stride % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)Wup % 16 == 0 &&
                (uintptr_t)Wdown % 16 == 0 && (uintptr_t)act % 16 == 0,
                "moe_grouped: inner sizes (K=%d, F=%d) must be multiples of 8 and operands 16-byte aligned", K, F);
    const int BM = zlm_moe_grouped_tile_rows(P, E);
    const int max_tiles = zlm_moe_grouped_max_tiles(P, E, BM);
    ZLM_REQUIRE(max_tiles <= 65535, "moe_grouped: too many tiles (%d)", max_tiles);
    int* perm = ints;
    int* inv = ints + P;
    int* tiles = ints + 2 * P;
    zlm_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)(3 * E + 2) * sizeof(int), st, idx, P, E, BM, max_tiles, 0, 0, perm,
               inv, tiles, tiles + max_tiles, tiles + 2 * max_tiles);
    int rc = zlm_check_launch("moe_sort");
    if (rc) return rc;
#define ZLM_MG(BM_, WM_, WN_)                                                                                         \
    do {                                                                                                              \
        rc = launch_grouped<BM_, 128, WM_, WN_, 0>(act, x, Wup, tiles, max_tiles, perm, wgt, top, F, K, x_stride, F,  \
                                                   scale_input, st);                                                  \
        if (rc) return rc;                                                                                            \
        rc = launch_grouped<BM_, 128, WM_, WN_, 1>(y, act, Wdown, tiles, max_tiles, perm, wgt, top, K, F, F, K,       \
                                                   scale_input, st);                                                  \
        if (rc) return rc;                                                                                            \
    } while (0)
    if (BM == 16) ZLM_MG(16, 1, 8);
    else if (BM == 64) ZLM_MG(64, 2, 4);
    else ZLM_MG(128, 2, 4);
#undef ZLM_MG
    zlm_launch(moe_combine_kernel, dim3(T), dim3(256), 0, st, stream, (const float*)y, (const int*)inv, (const float*)nullptr, top, K,
               (const __nv_bfloat16*)nullptr, 0, (const float*)nullptr);
    return zlm_check_launch("moe_combine");
}

// ---------------------------------------------------------------------------- the pieces, for the tcgen05 grouped product
// Rows in tiles of 128 with every expert's rows starting at a tile (padded): ints = perm [max_tiles * 128] (-1: an
// empty row) | inv [P] | tile table [3 * max_tiles]; the table's first part is what zlm_gemm_tc_grouped reads.
extern "C" int zlm_moe_sort_padded(const int* idx, int P, int E, int max_tiles, int* ints, cudaStream_t st) {
    ZLM_REQUIRE(P > 0 && E > 0 && E <= 2048 && max_tiles > 0, "moe_sort: pairs=%d experts=%d tiles=%d", P, E, max_tiles);
    int* perm = ints;
    int* inv = ints + (size_t)max_tiles * 128;
    int* tiles = inv + P;
    zlm_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)(3 * E + 2) * sizeof(int), st, idx, P, E, 128, max_tiles, 1, 1, perm,
               inv, tiles, tiles + max_tiles, tiles + 2 * max_tiles);
    return zlm_check_launch("moe_sort");
}

// xs[row, :] = bf16(w * x[token(row), :]) for the sorted, padded rows (zeros in empty rows); w the pair's weight
// if scale (the weight on the expert's input), else 1
__global__ void __launch_bounds__(256)
moe_gather_kernel(__nv_bfloat16* __restrict__ xs, const __nv_bfloat16* __restrict__ x, int x_stride,
                  const int* __restrict__ perm, const float* __restrict__ wgt, int top, int K, int scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    if (!ZLM_CHK(perm + row, 4)) return;
    const int pair = perm[row];
    __nv_bfloat16* dst = xs + (size_t)row * K;
    if (pair < 0) {
        for (int c = threadIdx.x; c < K / 8; c += blockDim.x)
            if (ZLM_CHK(dst + c * 8, 16)) *(uint4*)(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const __nv_bfloat16* src = x + (size_t)(pair / top) * x_stride;
    const float w = (scale && ZLM_CHK(wgt + pair, 4)) ? wgt[pair] : 1.0f;
    for (int c = threadIdx.x; c < K / 8; c += blockDim.x) {
        if (!ZLM_CHK(src + c * 8, 16) || !ZLM_CHK(dst + c * 8, 16)) continue;
        uint4 v = *(const uint4*)(src + c * 8);
        if (scale) {
            unsigned* u = (unsigned*)&v;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                u[i] = pack_bf16(__uint_as_float(u[i] << 16) * w, __uint_as_float(u[i] & 0xffff0000u) * w);
        }
        *(uint4*)(dst + c * 8) = v;
    }
}

extern "C" int zlm_moe_gather(void* xs, const void* x, int x_stride, const int* perm, const float* wgt, int rows, int top,
                              int K, int scale, cudaStream_t st) {
    if (rows == 0) return ZLM_OK;
    ZLM_REQUIRE(K % 8 == 0 && x_stride % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)xs % 16 == 0,
                "moe_gather: K=%d and the row stride must be multiples of 8, operands 16-byte aligned", K);
    zlm_launch(moe_gather_kernel, dim3(rows), dim3(256), 0, st, (__nv_bfloat16*)xs, (const __nv_bfloat16*)x, x_stride, perm, wgt,
               top, K, scale);
    return zlm_check_launch("moe_gather");
}

// stream[t, :] += sum_j (wgt[t, j] or 1) * y[inv[t, j], :]; a pair with inv < 0 (an identity expert, dropped by the sort)
// adds xw[t, j] * x[t, :] if x (bf16 [T, x_stride]) is given
extern "C" int zlm_moe_combine(float* stream, const float* y, const int* inv, const float* wgt, int T, int top, int N,
                               const void* x, int x_stride, const float* xw, cudaStream_t st) {
    if (T == 0) return ZLM_OK;
    ZLM_REQUIRE(!x || xw, "moe_combine: identity experts need their weights");
    zlm_launch(moe_combine_kernel, dim3(T), dim3(256), 0, st, stream, y, inv, wgt, top, N, (const __nv_bfloat16*)x, x_stride, xw);
    return zlm_check_launch("moe_combine");
}

ZLM_TRANSLATION_UNIT(moe_grouped)
