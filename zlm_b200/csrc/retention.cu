// Retention: linear attention with one fixed decay per head, no softmax and no denominator.
//
//   q_t, k_t = rot(q_t), rot(k_t) * k_scale      rotation of the first n_rot coordinates of a head, coordinate i
//                                                with i + n_rot/2, by the angle pos * inv_freq[i]
//   S_t = decay_h * S_(t-1) + k_t v_t^T          [dim][vdim] per head and sequence, fp32, kept in the sequence's state
//   o_t = S_t^T q_t                              fp32
//
// q, k, v are columns of one fused projection [T][ld] in the compute element type; everything after the
// projection (angles, rotated q and k, the decay, the state, o) is fp32 in both element types.
//
// The columns of the state are independent: a thread holds DPT rows of one column in registers, the `ds`
// threads that share a column are neighbouring lanes and add their parts of o by shuffles.  A block takes
// 128 / ds columns of one head of one sequence and walks the sequence's tokens in order, RT_CHUNK at a time:
// the chunk's rotated q and k and its v columns are staged in shared memory by the whole block.
//
// Long prompts, three kernels (retention_parts): the sequence is cut into pieces of `piece` tokens;
//   1. every piece runs the recurrence from a zero state (the same code): its local outputs, and the state
//      it would leave, A_c
//   2. the pieces' states are chained: S_c = decay^len_c * S_(c-1) + A_c   (S_(-1) is the sequence's state)
//   3. every piece adds what the state before it contributes: o_t += decay^(t - t0 + 1) * S_(c-1)^T q_t
// so that the pieces run side by side; the sums are the same up to their order.
#include "common.cuh"

#define RT_THREADS 128
#define RT_CHUNK 16

// rotated coordinate i of a head's vector x (fp32 angle)
template <typename TA>
__device__ __forceinline__ float rotated(const TA* __restrict__ x, int i, int n_rot, const float* __restrict__ inv_freq, int pos) {
    if (i >= n_rot) return to_f32(x[i]);
    const int half = n_rot >> 1;
    const int f = i < half ? i : i - half;
    float sn, cs;
    sincosf((float)pos * inv_freq[f], &sn, &cs);
    const float u = to_f32(x[f]), v = to_f32(x[f + half]);
    return i < half ? u * cs - v * sn : v * cs + u * sn;
}

// MODE 0: the whole recurrence from the sequence's state (reads and writes `state`).
// MODE 1: a piece from a zero state; its final state goes to part_state [pieces][H][D][V].
// MODE 2: o += decay^(j+1) * S_before^T q for a piece, S_before from chain [pieces][H][D][V] (the state before piece c).
template <typename TA, int DPT, int MODE>
__global__ void __launch_bounds__(RT_THREADS)
retention_kernel(float* __restrict__ o, const TA* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                 const float* __restrict__ inv_freq, int n_rot, const float* __restrict__ decay, float* __restrict__ state,
                 const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                 const int* __restrict__ piece_seq, const int* __restrict__ piece_first, int piece, int H, int D, int V,
                 int ds, float k_scale) {
    extern __shared__ float sm[];
    float* qs = sm;                          // [RT_CHUNK][D]
    float* ks = qs + RT_CHUNK * D;           // [RT_CHUNK][D]
    const int cols = RT_THREADS / ds;
    float* vs = ks + RT_CHUNK * D;           // [RT_CHUNK][cols]
    pdl_launch_dependents();
    const int tid = threadIdx.x, h = blockIdx.y;
    const int col = blockIdx.x * cols + tid / ds, part = tid % ds;
    pdl_wait();
    int r, first, n;                          // sequence, first token of this block's run within the step, tokens
    if (MODE == 0) {
        r = blockIdx.z;
        first = 0;
        n = cu_seqlens[r + 1] - cu_seqlens[r];
    } else {
        r = piece_seq[blockIdx.z];
        first = piece_first[blockIdx.z];
        n = min(piece, cu_seqlens[r + 1] - cu_seqlens[r] - first);
    }
    const int row0 = cu_seqlens[r] + first, pos0 = seq_start[r] + first;
    const float d = decay[h];
    float S[DPT];
    const bool live = col < V;
    float* sp = nullptr;
    if (MODE == 0) sp = state + ((size_t)seq_slot[r] * H + h) * D * V;
    else sp = state + ((size_t)blockIdx.z * H + h) * D * V;       // MODE 1: part_state (written); MODE 2: chain (read)
#pragma unroll
    for (int j = 0; j < DPT; ++j) {
        const int i = part * DPT + j;
        S[j] = (MODE != 1 && live && i < D && ZLM_CHK(sp + (size_t)i * V + col, 4)) ? sp[(size_t)i * V + col] : 0.f;
    }
    float dp = d;                              // MODE 2: decay^(j+1)
    for (int c0 = 0; c0 < n; c0 += RT_CHUNK) {
        const int cn = min(RT_CHUNK, n - c0);
        __syncthreads();
        for (int idx = tid; idx < cn * D; idx += RT_THREADS) {
            const int tt = idx / D, i = idx % D;
            const TA* row = proj + (size_t)(row0 + c0 + tt) * ld + (size_t)h * D;
            if (!ZLM_CHK(row + q_off, (size_t)D * sizeof(TA)) || !ZLM_CHK(row + k_off, (size_t)D * sizeof(TA))) continue;
            qs[tt * D + i] = rotated(row + q_off, i, n_rot, inv_freq, pos0 + c0 + tt);
            if (MODE != 2) ks[tt * D + i] = rotated(row + k_off, i, n_rot, inv_freq, pos0 + c0 + tt) * k_scale;
        }
        if (MODE != 2)
            for (int idx = tid; idx < cn * cols; idx += RT_THREADS) {
                const int tt = idx / cols, cc = idx % cols, gc = blockIdx.x * cols + cc;
                const TA* vp = proj + (size_t)(row0 + c0 + tt) * ld + v_off + (size_t)h * V + gc;
                vs[tt * cols + cc] = (gc < V && ZLM_CHK(vp, sizeof(TA))) ? to_f32(*vp) : 0.f;
            }
        __syncthreads();
        for (int tt = 0; tt < cn; ++tt) {
            float acc = 0.f;
            const float* qr = qs + tt * D + part * DPT;
            if (MODE == 2) {
#pragma unroll
                for (int j = 0; j < DPT; ++j)
                    if (part * DPT + j < D) acc = fmaf(S[j], qr[j], acc);
                acc *= dp;
                dp *= d;
            } else {
                const float* kr = ks + tt * D + part * DPT;
                const float v = vs[tt * cols + tid / ds];
#pragma unroll
                for (int j = 0; j < DPT; ++j)
                    if (part * DPT + j < D) {
                        S[j] = fmaf(d, S[j], kr[j] * v);
                        acc = fmaf(S[j], qr[j], acc);
                    }
            }
            for (int off = ds >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            float* op = o + (size_t)(row0 + c0 + tt) * H * V + (size_t)h * V + col;
            if (part == 0 && live && ZLM_CHK(op, 4)) {
                if (MODE == 2) *op += acc;
                else *op = acc;
            }
        }
    }
    if (MODE != 2 && live) {
#pragma unroll
        for (int j = 0; j < DPT; ++j) {
            const int i = part * DPT + j;
            if (i < D && ZLM_CHK(sp + (size_t)i * V + col, 4)) sp[(size_t)i * V + col] = S[j];
        }
    }
}

// chains the pieces' states of one sequence: before[c] = S_(c-1), S_c = decay^len_c * S_(c-1) + part[c]; the last S
// becomes the sequence's state.  grid (ceil(D*V / 256), H, R); the pieces of sequence r are seq_piece0[r] .. seq_piece0[r+1]-1
// and `part_state` is overwritten in place by `before`.
__global__ void __launch_bounds__(256)
retention_chain_kernel(float* __restrict__ part_state, float* __restrict__ state, const float* __restrict__ decay,
                       const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                       const int* __restrict__ seq_piece0, int piece, int H, int DV) {
    pdl_launch_dependents();
    const int e = blockIdx.x * 256 + threadIdx.x, h = blockIdx.y, r = blockIdx.z;
    pdl_wait();
    if (e >= DV) return;
    const int n = cu_seqlens[r + 1] - cu_seqlens[r];
    const int p0 = seq_piece0[r], np = seq_piece0[r + 1] - p0;
    float* sp = state + ((size_t)seq_slot[r] * H + h) * DV + e;
    if (!ZLM_CHK(sp, 4)) return;
    float S = *sp;
    const float d = decay[h];
    for (int c = 0; c < np; ++c) {
        float* pp = part_state + ((size_t)(p0 + c) * H + h) * DV + e;
        if (!ZLM_CHK(pp, 4)) continue;
        const int len = min(piece, n - c * piece);
        const float a = *pp;
        *pp = S;
        S = fmaf(powf(d, (float)len), S, a);
    }
    *sp = S;
}

static int retention_dpt(int D, int* ds) {
    // rows of a column per thread: 32 where that leaves at most 8 threads a column, else more
    int dpt = D <= 32 ? 32 : (D <= 256 ? 32 : 64);
    int n = (D + dpt - 1) / dpt, p = 1;
    while (p < n) p <<= 1;
    *ds = p;
    return dpt;
}

template <typename TA, int MODE>
static int launch_retention(dim3 grid, size_t smem, cudaStream_t st, int dpt, float* o, const void* proj, int ld, int q_off,
                            int k_off, int v_off, const float* inv_freq, int n_rot, const float* decay, float* state,
                            const int* cu_seqlens, const int* seq_slot, const int* seq_start, const int* piece_seq,
                            const int* piece_first, int piece, int H, int D, int V, int ds, float k_scale) {
#define ZLM_RT_LAUNCH(DPT)                                                                                                \
    {                                                                                                                     \
        auto kern = retention_kernel<TA, DPT, MODE>;                                                                      \
        static bool attr_set_dev[64] = {}; bool& attr_set = attr_set_dev[zlm_device_index()];                             \
        if (!attr_set) {                                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);          \
            if (e != cudaSuccess) {                                                                                       \
                zlm_set_error("retention: cannot reserve shared memory: %s", cudaGetErrorString(e));                      \
                return ZLM_ERR_CUDA;                                                                                      \
            }                                                                                                             \
            attr_set = true;                                                                                              \
        }                                                                                                                 \
        zlm_launch(kern, grid, dim3(RT_THREADS), smem, st, o, (const TA*)proj, ld, q_off, k_off, v_off, inv_freq, n_rot,   \
                   decay, state, cu_seqlens, seq_slot, seq_start, piece_seq, piece_first, piece, H, D, V, ds, k_scale);    \
    }
    if (dpt == 32) ZLM_RT_LAUNCH(32)
    else ZLM_RT_LAUNCH(64)
#undef ZLM_RT_LAUNCH
    return ZLM_OK;
}

static int retention_check(int H, int D, int V, int n_rot, int R) {
    ZLM_REQUIRE(H > 0 && H <= 65535 && D > 0 && D <= 1024 && V > 0 && R <= 65535, "retention: %d heads of %d x %d, %d sequences", H, D, V, R);
    ZLM_REQUIRE(n_rot >= 0 && n_rot % 2 == 0 && n_rot <= D, "retention: %d rotated coordinates of %d", n_rot, D);
    return ZLM_OK;
}

// o [T][H*V] fp32; proj [T][ld] with q at column q_off (H heads of D), k at k_off, v at v_off (H heads of V);
// state [slots][H][D][V] fp32 (zero for a new sequence)
extern "C" int zlm_retention(float* o, const void* proj, int ld, int q_off, int k_off, int v_off, int dtype,
                             const float* inv_freq, int n_rot, const float* decay, float* state, const int* cu_seqlens,
                             const int* seq_slot, const int* seq_start, int R, int H, int D, int V, float k_scale,
                             cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    int rc = retention_check(H, D, V, n_rot, R);
    if (rc) return rc;
    int ds;
    const int dpt = retention_dpt(D, &ds);
    const int cols = RT_THREADS / ds;
    const size_t smem = (size_t)RT_CHUNK * (2 * D + cols) * sizeof(float);
    const dim3 grid((V + cols - 1) / cols, H, R);
    if (dtype == ZLM_DTYPE_F32)
        rc = launch_retention<float, 0>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq, n_rot, decay, state,
                                        cu_seqlens, seq_slot, seq_start, nullptr, nullptr, 0, H, D, V, ds, k_scale);
    else if (dtype == ZLM_DTYPE_BF16)
        rc = launch_retention<__nv_bfloat16, 0>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq, n_rot, decay,
                                                state, cu_seqlens, seq_slot, seq_start, nullptr, nullptr, 0, H, D, V, ds, k_scale);
    else
        ZLM_REQUIRE(false, "retention: unsupported dtype %d", dtype);
    if (rc) return rc;
    return zlm_check_launch("retention");
}

// The same for long prompts, in pieces of `piece` tokens that run side by side.  The host lists the pieces:
// piece_seq / piece_first [pieces] (the sequence of a piece and its first token within the sequence's tokens of
// this step), seq_piece0 [R + 1] (a sequence's first piece); part_state is scratch of pieces * H * D * V floats.
extern "C" int zlm_retention_parts(float* o, const void* proj, int ld, int q_off, int k_off, int v_off, int dtype,
                                   const float* inv_freq, int n_rot, const float* decay, float* state,
                                   const int* cu_seqlens, const int* seq_slot, const int* seq_start, int R,
                                   const int* piece_seq, const int* piece_first, const int* seq_piece0, int pieces, int piece,
                                   float* part_state, int H, int D, int V, float k_scale, cudaStream_t st) {
    if (R == 0 || pieces == 0) return ZLM_OK;
    int rc = retention_check(H, D, V, n_rot, R);
    if (rc) return rc;
    ZLM_REQUIRE(piece > 0 && pieces <= 65535 && part_state, "retention: %d pieces of %d tokens", pieces, piece);
    int ds;
    const int dpt = retention_dpt(D, &ds);
    const int cols = RT_THREADS / ds;
    const size_t smem = (size_t)RT_CHUNK * (2 * D + cols) * sizeof(float);
    const dim3 grid((V + cols - 1) / cols, H, pieces);
    for (int mode = 1; mode <= 2; ++mode) {
        if (dtype == ZLM_DTYPE_F32) {
            rc = mode == 1 ? launch_retention<float, 1>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq, n_rot, decay,
                                                        part_state, cu_seqlens, seq_slot, seq_start, piece_seq, piece_first, piece,
                                                        H, D, V, ds, k_scale)
                           : launch_retention<float, 2>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq, n_rot, decay,
                                                        part_state, cu_seqlens, seq_slot, seq_start, piece_seq, piece_first, piece,
                                                        H, D, V, ds, k_scale);
        } else if (dtype == ZLM_DTYPE_BF16) {
            rc = mode == 1 ? launch_retention<__nv_bfloat16, 1>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq,
                                                                n_rot, decay, part_state, cu_seqlens, seq_slot, seq_start,
                                                                piece_seq, piece_first, piece, H, D, V, ds, k_scale)
                           : launch_retention<__nv_bfloat16, 2>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq,
                                                                n_rot, decay, part_state, cu_seqlens, seq_slot, seq_start,
                                                                piece_seq, piece_first, piece, H, D, V, ds, k_scale);
        } else {
            ZLM_REQUIRE(false, "retention: unsupported dtype %d", dtype);
        }
        if (rc) return rc;
        rc = zlm_check_launch("retention_parts");
        if (rc) return rc;
        if (mode == 1) {
            zlm_launch(retention_chain_kernel, dim3((D * V + 255) / 256, H, R), dim3(256), 0, st, part_state, state, decay,
                       cu_seqlens, seq_slot, seq_piece0, piece, H, D * V);
            rc = zlm_check_launch("retention_chain");
            if (rc) return rc;
        }
    }
    return ZLM_OK;
}

ZLM_TRANSLATION_UNIT(retention)
