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
// The columns of the state are independent: a thread holds DPT rows of four columns in registers, the `ds`
// threads that share the columns are neighbouring lanes and add their parts of o by shuffles.  A block takes
// 4 * 128 / ds columns of one head of one sequence and walks the sequence's tokens in order, RT_CHUNK at a time:
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
#define RT_CHUNK 64          // tokens staged at a time, at most (a piece of a long prompt)

// MODE 0: the whole recurrence from the sequence's state (reads and writes `state`).
// MODE 1: a piece from a zero state; its final state goes to part_state [pieces][H][D][V].
// MODE 2: o += decay^(j+1) * S_before^T q for a piece, S_before from chain [pieces][H][D][V] (the state before piece c).
//
// A thread holds a tile of DPT rows x RT_CPT columns of the state, so that a staged q or k value is used for
// RT_CPT columns and a v value for DPT rows (one column a thread had every thread read all of q and k from shared
// memory for every token, and the shared-memory pipe, not the arithmetic, set the time).  The `ds` threads that
// share a tile's columns are neighbouring lanes; their segments of a staged row lie DPT + 4 floats apart, so that
// their 16-byte reads fall into different banks.
#define RT_CPT 4
template <typename TA, int DPT, int MODE>
__global__ void __launch_bounds__(RT_THREADS)
retention_kernel(float* __restrict__ o, const TA* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                 const float* __restrict__ inv_freq, int n_rot, const float* __restrict__ decay, float* __restrict__ state,
                 const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                 int maxp, int piece, int H, int D, int V,
                 int ds, float k_scale, const float* __restrict__ table, int T, int chunk) {
    extern __shared__ __align__(16) float sm[];
    const int DP = ds * (DPT + 4);           // a staged row: ds segments of DPT values, 4 floats of padding after each
    float* qs = sm;                          // [chunk][DP]
    float* ks = qs + chunk * DP;             // [chunk][DP]
    const int cols = RT_THREADS / ds * RT_CPT;
    float* vs = ks + chunk * DP;             // [chunk][cols]
    pdl_launch_dependents();
    const int tid = threadIdx.x, h = blockIdx.y;
    const int grp = tid / ds, part = tid % ds;
    const int col0 = blockIdx.x * cols + grp * RT_CPT;
    pdl_wait();
    int r, first, n;                          // sequence, first token of this block's run within the step, tokens
    if (MODE == 0) {
        r = blockIdx.z;
        first = 0;
        n = cu_seqlens[r + 1] - cu_seqlens[r];
    } else {
        // piece blockIdx.z % maxp of sequence blockIdx.z / maxp (maxp: the pieces of the step's longest sequence)
        r = blockIdx.z / maxp;
        first = (blockIdx.z % maxp) * piece;
        n = min(piece, cu_seqlens[r + 1] - cu_seqlens[r] - first);
        if (n <= 0) return;
    }
    const int row0 = cu_seqlens[r] + first, pos0 = seq_start[r] + first;
    const float d = decay[h];
    // the tile, two neighbouring rows a register pair (packed fp32 arithmetic: the pairs of q and k come straight
    // from their 16-byte reads)
    float2 S[DPT / 2][RT_CPT];
    float* sp = nullptr;
    if (MODE == 0) sp = state + ((size_t)seq_slot[r] * H + h) * D * V;
    else sp = state + ((size_t)blockIdx.z * H + h) * D * V;       // MODE 1: part_state (written); MODE 2: chain (read)
    const bool v4 = (V & 3) == 0 && col0 + RT_CPT <= V;             // the tile's columns as one 16-byte access
#pragma unroll
    for (int jj = 0; jj < DPT / 2; ++jj) {
        float t[2][RT_CPT];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int i = part * DPT + 2 * jj + e;
#pragma unroll
            for (int c = 0; c < RT_CPT; ++c) t[e][c] = 0.f;
            if (MODE == 1 || i >= D) continue;
            const float* src = sp + (size_t)i * V + col0;
            if (v4 && ZLM_CHK(src, 16)) {
                const float4 a = *(const float4*)src;
                t[e][0] = a.x; t[e][1] = a.y; t[e][2] = a.z; t[e][3] = a.w;
            } else {
#pragma unroll
                for (int c = 0; c < RT_CPT; ++c)
                    if (col0 + c < V && ZLM_CHK(src + c, 4)) t[e][c] = src[c];
            }
        }
#pragma unroll
        for (int c = 0; c < RT_CPT; ++c) S[jj][c] = make_float2(t[0][c], t[1][c]);
    }
    float dp = d;                              // MODE 2: decay^(j+1)
    const int half = n_rot >> 1;
    for (int c0 = 0; c0 < n; c0 += chunk) {
        const int cn = min(chunk, n - c0);
        __syncthreads();
        // the chunk's q and k, rotated: a thread turns a pair (f, f + half) of a token at a time, so that the pair and
        // its cosine and sine are read once; the loads of several pairs are in flight together
#pragma unroll 8
        for (int idx = tid; idx < cn * half; idx += RT_THREADS) {
            const int tt = idx / half, f = idx % half;
            const int rowi = row0 + c0 + tt;
            const TA* row = proj + (size_t)rowi * ld + (size_t)h * D;
            if (!ZLM_CHK(row + q_off, (size_t)D * sizeof(TA)) || !ZLM_CHK(row + k_off, (size_t)D * sizeof(TA))) continue;
            float sn, cs;
            if (table) {
                cs = table[(size_t)f * T + rowi];
                sn = table[(size_t)(half + f) * T + rowi];
            } else {
                sincosf((float)(pos0 + c0 + tt) * inv_freq[f], &sn, &cs);
            }
            const int i1 = f + half;
            const int a0 = tt * DP + (f / DPT) * (DPT + 4) + f % DPT, a1 = tt * DP + (i1 / DPT) * (DPT + 4) + i1 % DPT;
            const float qu = to_f32(row[q_off + f]), qv = to_f32(row[q_off + i1]);
            qs[a0] = qu * cs - qv * sn;
            qs[a1] = qv * cs + qu * sn;
            if (MODE != 2) {
                const float ku = to_f32(row[k_off + f]), kv = to_f32(row[k_off + i1]);
                ks[a0] = (ku * cs - kv * sn) * k_scale;
                ks[a1] = (kv * cs + ku * sn) * k_scale;
            }
        }
        // what lies beyond the rotated coordinates passes as it is
#pragma unroll 4
        for (int idx = tid; idx < cn * (D - n_rot); idx += RT_THREADS) {
            const int tt = idx / (D - n_rot), i = n_rot + idx % (D - n_rot);
            const TA* row = proj + (size_t)(row0 + c0 + tt) * ld + (size_t)h * D;
            if (!ZLM_CHK(row + q_off + i, sizeof(TA)) || !ZLM_CHK(row + k_off + i, sizeof(TA))) continue;
            const int at = tt * DP + (i / DPT) * (DPT + 4) + i % DPT;
            qs[at] = to_f32(row[q_off + i]);
            if (MODE != 2) ks[at] = to_f32(row[k_off + i]) * k_scale;
        }
        // rows of the tiles beyond the head's own stay zero: the walk below asks no row whether it exists
        for (int idx = tid; idx < cn * (ds * DPT - D); idx += RT_THREADS) {
            const int tt = idx / (ds * DPT - D), i = D + idx % (ds * DPT - D);
            const int at = tt * DP + (i / DPT) * (DPT + 4) + i % DPT;
            qs[at] = 0.f;
            ks[at] = 0.f;
        }
        if (MODE != 2) {
#pragma unroll 8
            for (int idx = tid; idx < cn * cols; idx += RT_THREADS) {
                const int tt = idx / cols, cc = idx % cols, gc = blockIdx.x * cols + cc;
                const TA* vp = proj + (size_t)(row0 + c0 + tt) * ld + v_off + (size_t)h * V + gc;
                vs[tt * cols + cc] = (gc < V && ZLM_CHK(vp, sizeof(TA))) ? to_f32(*vp) : 0.f;
            }
        } else {
            // the outputs that the pieces' own walks left, to which this pass adds: staged like the values, so that the
            // walk below does not wait for global memory at every token
#pragma unroll 8
            for (int idx = tid; idx < cn * cols; idx += RT_THREADS) {
                const int tt = idx / cols, cc = idx % cols, gc = blockIdx.x * cols + cc;
                const float* op = o + (size_t)(row0 + c0 + tt) * H * V + (size_t)h * V + gc;
                vs[tt * cols + cc] = (gc < V && ZLM_CHK(op, 4)) ? *op : 0.f;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < cn; ++tt) {
            float2 acc2[RT_CPT];
            float2 vv[RT_CPT];
#pragma unroll
            for (int c = 0; c < RT_CPT; ++c) acc2[c] = vv[c] = make_float2(0.f, 0.f);
            const float* qr = qs + tt * DP + part * (DPT + 4);
            const float* kr = ks + tt * DP + part * (DPT + 4);
            if (MODE != 2) {
                const float4 a = *(const float4*)(vs + tt * cols + grp * RT_CPT);
                vv[0] = make_float2(a.x, a.x); vv[1] = make_float2(a.y, a.y);
                vv[2] = make_float2(a.z, a.z); vv[3] = make_float2(a.w, a.w);
            }
            const float2 d2 = make_float2(d, d);
            // S = d S + k v and o += S q, two rows an instruction (each element rounded as fmaf and a product would
            // round it); acc2 holds the sums over a thread's even and odd rows
#pragma unroll
            for (int j = 0; j < DPT; j += 4) {
                const float4 qa = *(const float4*)(qr + j);
                const float2 q2[2] = {make_float2(qa.x, qa.y), make_float2(qa.z, qa.w)};
                float2 k2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
                if (MODE != 2) {
                    const float4 ka = *(const float4*)(kr + j);
                    k2[0] = make_float2(ka.x, ka.y);
                    k2[1] = make_float2(ka.z, ka.w);
                }
#pragma unroll
                for (int e = 0; e < 2; ++e)
#pragma unroll
                    for (int c = 0; c < RT_CPT; ++c) {
                        if (MODE != 2) S[j / 2 + e][c] = __ffma2_rn(d2, S[j / 2 + e][c], __fmul2_rn(k2[e], vv[c]));
                        acc2[c] = __ffma2_rn(S[j / 2 + e][c], q2[e], acc2[c]);
                    }
            }
            float acc[RT_CPT];
#pragma unroll
            for (int c = 0; c < RT_CPT; ++c) acc[c] = (acc2[c].x + acc2[c].y) * (MODE == 2 ? dp : 1.0f);
            if (MODE == 2) dp *= d;
            // the ds lanes of a tile add up their parts; while they do, the columns are dealt out among them (half of
            // the lanes go on with columns 0-1, half with 2-3, then one column each), so that the sums cost 4 shuffles
            // where 4 x log2(ds) would be the plain way.  `mine` is the first column a lane ends up with, `have` how many.
            int mine = 0, have = RT_CPT;
            if (ds >= 2) {
                const int off = ds >> 1;
                const bool up = (part & off) != 0;
                const float s0 = up ? acc[0] : acc[2], s1 = up ? acc[1] : acc[3];
                const float r0 = __shfl_xor_sync(0xffffffffu, s0, off), r1 = __shfl_xor_sync(0xffffffffu, s1, off);
                acc[0] = (up ? acc[2] : acc[0]) + r0;
                acc[1] = (up ? acc[3] : acc[1]) + r1;
                mine = up ? 2 : 0;
                have = 2;
            }
            if (ds >= 4) {
                const int off = ds >> 2;
                const bool up = (part & off) != 0;
                const float r0 = __shfl_xor_sync(0xffffffffu, up ? acc[0] : acc[1], off);
                acc[0] = (up ? acc[1] : acc[0]) + r0;
                mine += up ? 1 : 0;
                have = 1;
                for (int o2 = ds >> 3; o2 > 0; o2 >>= 1) acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], o2);
            }
            // the lanes whose lower bits are zero write
            const bool writer = ds < 8 || (part & ((ds >> 2) - 1)) == 0;
            float* op = o + (size_t)(row0 + c0 + tt) * H * V + (size_t)h * V + col0 + mine;
            if (writer) {
#pragma unroll
                for (int c = 0; c < RT_CPT; ++c)
                    if (c < have && col0 + mine + c < V && ZLM_CHK(op + c, 4))
                        op[c] = MODE == 2 ? vs[tt * cols + grp * RT_CPT + mine + c] + acc[c] : acc[c];
            }
        }
    }
    if (MODE != 2) {
#pragma unroll
        for (int jj = 0; jj < DPT / 2; ++jj)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int i = part * DPT + 2 * jj + e;
                if (i >= D) continue;
                float* dst = sp + (size_t)i * V + col0;
                const float t[RT_CPT] = {e ? S[jj][0].y : S[jj][0].x, e ? S[jj][1].y : S[jj][1].x, e ? S[jj][2].y : S[jj][2].x,
                                         e ? S[jj][3].y : S[jj][3].x};
                if (v4 && ZLM_CHK(dst, 16)) {
                    *(float4*)dst = make_float4(t[0], t[1], t[2], t[3]);
                } else {
#pragma unroll
                    for (int c = 0; c < RT_CPT; ++c)
                        if (col0 + c < V && ZLM_CHK(dst + c, 4)) dst[c] = t[c];
                }
            }
    }
}

// chains the pieces' states of one sequence: before[c] = S_(c-1), S_c = decay^len_c * S_(c-1) + part[c]; the last S
// becomes the sequence's state.  grid (ceil(D*V / 256), H, R); the pieces of sequence r are r * maxp .. and `part_state`
// is overwritten in place by `before`.
__global__ void __launch_bounds__(256)
retention_chain_kernel(float* __restrict__ part_state, float* __restrict__ state, const float* __restrict__ decay,
                       const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, int maxp, int piece, int H,
                       int DV) {
    pdl_launch_dependents();
    const int e = blockIdx.x * 256 + threadIdx.x, h = blockIdx.y, r = blockIdx.z;
    pdl_wait();
    if (e >= DV) return;
    const int n = cu_seqlens[r + 1] - cu_seqlens[r];
    const int p0 = r * maxp, np = (n + piece - 1) / piece;
    float* sp = state + ((size_t)seq_slot[r] * H + h) * DV + e;
    if (!ZLM_CHK(sp, 4)) return;
    float S = *sp;
    const float d = decay[h];
    const float dl = powf(d, (float)piece);            // every piece but the last is whole
    for (int c0 = 0; c0 < np; c0 += 8) {
        // eight pieces' states at a time: their loads do not wait for each other
        float a[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float* pp = part_state + ((size_t)(p0 + c0 + u) * H + h) * DV + e;
            a[u] = (c0 + u < np && ZLM_CHK(pp, 4)) ? *pp : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int c = c0 + u;
            if (c >= np) break;
            float* pp = part_state + ((size_t)(p0 + c) * H + h) * DV + e;
            if (ZLM_CHK(pp, 4)) *pp = S;
            const int len = min(piece, n - c * piece);
            S = fmaf(len == piece ? dl : powf(d, (float)len), S, a[u]);
        }
    }
    *sp = S;
}

static int retention_dpt(int D, int* ds) {
    // rows of the state a thread holds (times four columns, all in registers): 16 where 32 lanes of 16 hold a head's
    // rows (about 110 registers a thread: four blocks an SM), else 32; heads of more than 1024 rows are refused
    int dpt = D <= 512 ? 16 : 32;
    int n = (D + dpt - 1) / dpt, p = 1;
    while (p < n) p <<= 1;
    *ds = p;
    return dpt;
}

template <typename TA, int MODE>
static int launch_retention(dim3 grid, size_t smem, cudaStream_t st, int dpt, float* o, const void* proj, int ld, int q_off,
                            int k_off, int v_off, const float* inv_freq, int n_rot, const float* decay, float* state,
                            const int* cu_seqlens, const int* seq_slot, const int* seq_start, int maxp, int piece, int H, int D,
                            int V, int ds, float k_scale, const float* table, int T, int chunk) {
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
                   decay, state, cu_seqlens, seq_slot, seq_start, maxp, piece, H, D, V, ds, k_scale,                      \
                   table, T, chunk);                                                                                      \
    }
    if (dpt == 32) ZLM_RT_LAUNCH(32)
    else ZLM_RT_LAUNCH(16)
#undef ZLM_RT_LAUNCH
    return ZLM_OK;
}

static int retention_check(int H, int D, int V, int n_rot, int R) {
    ZLM_REQUIRE(H > 0 && H <= 65535 && D > 0 && D <= 1024 && V > 0 && R <= 65535, "retention: %d heads of %d x %d, %d sequences", H, D, V, R);
    ZLM_REQUIRE(n_rot >= 0 && n_rot % 2 == 0 && n_rot <= D, "retention: %d rotated coordinates of %d", n_rot, D);
    return ZLM_OK;
}

// o [T][H*V] fp32; proj [T][ld] with q at column q_off (H heads of D), k at k_off, v at v_off (H heads of V);
// state [slots][H][D][V] fp32 (zero for a new sequence); table: the step's cosines and sines [2][n_rot/2][T] if they were
// computed beforehand (else the kernel forms them from inv_freq)
extern "C" int zlm_retention(float* o, const void* proj, int ld, int q_off, int k_off, int v_off, int dtype,
                             const float* inv_freq, int n_rot, const float* decay, float* state, const int* cu_seqlens,
                             const int* seq_slot, const int* seq_start, int R, int H, int D, int V, float k_scale,
                             const float* table, int T, int max_new, cudaStream_t st) {
    if (R == 0) return ZLM_OK;
    int rc = retention_check(H, D, V, n_rot, R);
    if (rc) return rc;
    int ds;
    const int dpt = retention_dpt(D, &ds);
    const int cols = RT_THREADS / ds * RT_CPT;
    // tokens staged at a time: as many as fit in about 56 KB (four blocks an SM), at least 4
    const size_t row_bytes = (size_t)(2 * ds * (dpt + 4) + cols) * sizeof(float);
    int chunk = (int)((56 * 1024) / row_bytes);
    chunk = chunk > RT_CHUNK ? RT_CHUNK : (chunk < 4 ? 4 : chunk);
    if (max_new > 0 && chunk > max_new) chunk = max_new;          // (the longest sequence of the step: a decode step stages one token)
    const size_t smem = (size_t)chunk * row_bytes;
    const dim3 grid((V + cols - 1) / cols, H, R);
    if (dtype == ZLM_DTYPE_F32)
        rc = launch_retention<float, 0>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq, n_rot, decay, state,
                                        cu_seqlens, seq_slot, seq_start, 0, 0, H, D, V, ds, k_scale, table, T, chunk);
    else if (dtype == ZLM_DTYPE_BF16)
        rc = launch_retention<__nv_bfloat16, 0>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq, n_rot, decay,
                                                state, cu_seqlens, seq_slot, seq_start, 0, 0, H, D, V, ds, k_scale, table, T, chunk);
    else
        ZLM_REQUIRE(false, "retention: unsupported dtype %d", dtype);
    if (rc) return rc;
    return zlm_check_launch("retention");
}

// The same for long prompts, in pieces of `piece` tokens that run side by side: maxp pieces a sequence (those of the
// step's longest one; a shorter sequence's last pieces are empty); part_state is scratch of R * maxp * H * D * V floats.
extern "C" int zlm_retention_parts(float* o, const void* proj, int ld, int q_off, int k_off, int v_off, int dtype,
                                   const float* inv_freq, int n_rot, const float* decay, float* state,
                                   const int* cu_seqlens, const int* seq_slot, const int* seq_start, int R, int maxp, int piece,
                                   float* part_state, int H, int D, int V, float k_scale, const float* table, int T,
                                   cudaStream_t st) {
    if (R == 0 || maxp == 0) return ZLM_OK;
    const long long pieces = (long long)R * maxp;
    int rc = retention_check(H, D, V, n_rot, R);
    if (rc) return rc;
    ZLM_REQUIRE(piece > 0 && pieces <= 65535 && part_state, "retention: %lld pieces of %d tokens", pieces, piece);
    int ds;
    const int dpt = retention_dpt(D, &ds);
    const int cols = RT_THREADS / ds * RT_CPT;
    // tokens staged at a time: as many as fit in about 56 KB (four blocks an SM), at least 4
    const size_t row_bytes = (size_t)(2 * ds * (dpt + 4) + cols) * sizeof(float);
    int chunk = (int)((56 * 1024) / row_bytes);
    chunk = chunk > RT_CHUNK ? RT_CHUNK : (chunk < 4 ? 4 : chunk);
    if (chunk > piece) chunk = piece;
    const size_t smem = (size_t)chunk * row_bytes;
    const dim3 grid((V + cols - 1) / cols, H, (unsigned)pieces);
    for (int mode = 1; mode <= 2; ++mode) {
        if (dtype == ZLM_DTYPE_F32) {
            rc = mode == 1 ? launch_retention<float, 1>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq, n_rot, decay,
                                                        part_state, cu_seqlens, seq_slot, seq_start, maxp, piece,
                                                        H, D, V, ds, k_scale, table, T, chunk)
                           : launch_retention<float, 2>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq, n_rot, decay,
                                                        part_state, cu_seqlens, seq_slot, seq_start, maxp, piece,
                                                        H, D, V, ds, k_scale, table, T, chunk);
        } else if (dtype == ZLM_DTYPE_BF16) {
            rc = mode == 1 ? launch_retention<__nv_bfloat16, 1>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq,
                                                                n_rot, decay, part_state, cu_seqlens, seq_slot, seq_start,
                                                                maxp, piece, H, D, V, ds, k_scale, table, T, chunk)
                           : launch_retention<__nv_bfloat16, 2>(grid, smem, st, dpt, o, proj, ld, q_off, k_off, v_off, inv_freq,
                                                                n_rot, decay, part_state, cu_seqlens, seq_slot, seq_start,
                                                                maxp, piece, H, D, V, ds, k_scale, table, T, chunk);
        } else {
            ZLM_REQUIRE(false, "retention: unsupported dtype %d", dtype);
        }
        if (rc) return rc;
        rc = zlm_check_launch("retention_parts");
        if (rc) return rc;
        if (mode == 1) {
            zlm_launch(retention_chain_kernel, dim3((D * V + 255) / 256, H, R), dim3(256), 0, st, part_state, state, decay,
                       cu_seqlens, seq_slot, maxp, piece, H, D * V);
            rc = zlm_check_launch("retention_chain");
            if (rc) return rc;
        }
    }
    return ZLM_OK;
}

ZLM_TRANSLATION_UNIT(retention)
