// Many small matrix products in one launch: C_g = A_g W_g^T for groups g that share a shape but not their
// weights. Two ways to say which rows belong to which group:
//
//   batched   every group has the same M rows; group g reads columns [g * a_gcs, g * a_gcs + K) of A's rows and
//             writes columns [g * c_gcs, g * c_gcs + N) of C's rows (the heads of an attention layer, each with a
//             matrix of its own); grid.z = groups.
//   routed    rows were sorted by group into tiles of BM positions (`tile_group[tile]` = the group of a tile, -1 =
//             unused tile; `a_rows[pos]` = the row of A at a sorted position, -1 = padding; `c_rows[pos]` = the row of
//             C it writes): the experts of a routed feed-forward. Positions without an indirection are their own row.
//
// W is [groups][N (or 2 N), K], K contiguous. With DUAL the weight of a group is [gate rows | up rows] and the result
// is act(A gate^T) * (A up^T). Accumulation is float32 with one FMA per k in the order k = 0..K-1 whatever the tile or
// the batch, so a row's result does not depend on what else is in the launch; inputs may be float32 or bfloat16.
#include "common.cuh"

namespace llmie {

struct GroupedArgs {
  const void* A; long long lda; long long a_gcs;
  const int* a_rows;
  const void* W; long long w_gs; long long ldw;
  void* C; long long ldc; long long c_gcs;
  const int* c_rows;
  const int* tile_group;
  int M, N, K, act;
};

constexpr int kGK = 16;

template <typename TA, typename TC, int BM, int BN, int TM, int TN, bool DUAL>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
grouped_gemm_kernel(const GroupedArgs p) {
  constexpr int kThreads = (BM / TM) * (BN / TN);
  __shared__ float As[kGK][BM + 4];
  __shared__ float Ws[DUAL ? 2 : 1][kGK][BN + 4];
  __shared__ int rowA[BM], rowC[BM];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int tile = blockIdx.y;
  int group = blockIdx.z;
  if (p.tile_group) {
    group = p.tile_group[tile];
    if (group < 0) return;
  }
  const int m0 = tile * BM, n0 = blockIdx.x * BN;
  for (int r = tid; r < BM; r += kThreads) {
    const int pos = m0 + r;
    int ra = -1, rc = -1;
    if (pos < p.M) {
      ra = p.a_rows ? p.a_rows[pos] : pos;
      rc = p.c_rows ? p.c_rows[pos] : pos;
      if (ra < 0 || rc < 0) ra = rc = -1;
    }
    rowA[r] = ra;
    rowC[r] = rc;
  }
  __syncthreads();
  const TA* A = reinterpret_cast<const TA*>(p.A) + (size_t)group * p.a_gcs;
  const TA* W = reinterpret_cast<const TA*>(p.W) + (size_t)group * p.w_gs;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  float acc[DUAL ? 2 : 1][TM][TN];
#pragma unroll
  for (int s = 0; s < (DUAL ? 2 : 1); ++s)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[s][i][j] = 0.f;

  for (int k0 = 0; k0 < p.K; k0 += kGK) {
    for (int idx = tid; idx < BM * kGK; idx += kThreads) {
      const int r = idx / kGK, c = idx % kGK;
      const int ra = rowA[r], gk = k0 + c;
      As[c][r] = (ra >= 0 && gk < p.K) ? to_f32(A[(size_t)ra * p.lda + gk]) : 0.f;
    }
    for (int idx = tid; idx < BN * kGK; idx += kThreads) {
      const int r = idx / kGK, c = idx % kGK;
      const int gn = n0 + r, gk = k0 + c;
      const bool ok = gn < p.N && gk < p.K;
      Ws[0][c][r] = ok ? to_f32(W[(size_t)gn * p.ldw + gk]) : 0.f;
      if (DUAL) Ws[DUAL ? 1 : 0][c][r] = ok ? to_f32(W[(size_t)(gn + p.N) * p.ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kGK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int s = 0; s < (DUAL ? 2 : 1); ++s) {
#pragma unroll
        for (int j = 0; j < TN; ++j) w[j] = Ws[s][kk][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[s][i][j] = fmaf(a[i], w[j], acc[s][i][j]);
      }
    }
    __syncthreads();
  }
  TC* C = reinterpret_cast<TC*>(p.C) + (size_t)group * p.c_gcs;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int rc = rowC[ty * TM + i];
    if (rc < 0) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= p.N) continue;
      float v = acc[0][i][j];
      if (DUAL) {
        // the gate is rounded to the activation type before the activation, as a separate product would leave it
        const float g = to_f32(from_f32<TC>(v)), u = to_f32(from_f32<TC>(acc[DUAL ? 1 : 0][i][j]));
        v = apply_act(g, p.act) * u;
      }
      C[(size_t)rc * p.ldc + gn] = from_f32<TC>(v);
    }
  }
}

template <typename TA, typename TC, bool DUAL>
static int launch_grouped(const GroupedArgs& p, int n_tiles_small, int n_tiles_big, int groups_z, bool small,
                          cudaStream_t stream) {
  if (small) {
    dim3 grid((p.N + 31) / 32, n_tiles_small, groups_z);
    if (grid.y > 65535 || grid.z > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
    launch_k(grouped_gemm_kernel<TA, TC, 16, 32, 2, 2, DUAL>, grid, dim3(128), 0, stream, p);
  } else {
    dim3 grid((p.N + 63) / 64, n_tiles_big, groups_z);
    if (grid.y > 65535 || grid.z > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
    launch_k(grouped_gemm_kernel<TA, TC, 64, 64, 4, 4, DUAL>, grid, dim3(256), 0, stream, p);
  }
  return LLMIE_OK;
}

}  // namespace llmie

using namespace llmie;

// Rows per tile of the two forms; the sort that prepares a routed call must use the same number.
extern "C" int llmie_grouped_gemm_tile_rows(int small) { return small ? 16 : 64; }

// A, W of in_dtype; C of out_dtype. `groups` > 0 with tile_group == null: the batched form over M rows. tile_group !=
// null: the routed form over `n_tiles` tiles of sorted positions (M = number of positions, padding included).
// `small` picks tiles of 16 rows (few rows per group) instead of 64. dual: W holds [gate | up], act is applied.
extern "C" int llmie_grouped_gemm_nt(const void* A, long long lda, long long a_gcs, const int* a_rows, const void* W,
                                     long long w_gs, long long ldw, void* C, long long ldc, long long c_gcs,
                                     const int* c_rows, const int* tile_group, int n_tiles, int groups, int M, int N,
                                     int K, int dual, int act, int small, int in_dtype, int out_dtype,
                                     cudaStream_t stream) {
  if (!A || !W || !C || M < 0 || N <= 0 || K <= 0 || lda < 0 || ldw < K || ldc < 0 || act < 0 || act > 4)
    return LLMIE_ERR_BAD_ARG;
  if (!tile_group && groups <= 0) return LLMIE_ERR_BAD_ARG;
  if (tile_group && n_tiles < 0) return LLMIE_ERR_BAD_ARG;
  if ((in_dtype != LLMIE_F32 && in_dtype != LLMIE_BF16) || (out_dtype != LLMIE_F32 && out_dtype != LLMIE_BF16))
    return LLMIE_ERR_DTYPE;
  if (in_dtype == LLMIE_F32 && out_dtype != LLMIE_F32) return LLMIE_ERR_DTYPE;
  if (M == 0 || (tile_group && n_tiles == 0)) return LLMIE_OK;
  GroupedArgs p{A, lda, a_gcs, a_rows, W, w_gs, ldw, C, ldc, c_gcs, c_rows, tile_group, M, N, K, act};
  const int bm = small ? 16 : 64;
  const int tiles = tile_group ? n_tiles : (M + bm - 1) / bm;
  const int gz = tile_group ? 1 : groups;
  int rc;
  if (in_dtype == LLMIE_F32)
    rc = dual ? launch_grouped<float, float, true>(p, tiles, tiles, gz, small, stream)
              : launch_grouped<float, float, false>(p, tiles, tiles, gz, small, stream);
  else if (out_dtype == LLMIE_F32)
    rc = dual ? launch_grouped<__nv_bfloat16, float, true>(p, tiles, tiles, gz, small, stream)
              : launch_grouped<__nv_bfloat16, float, false>(p, tiles, tiles, gz, small, stream);
  else
    rc = dual ? launch_grouped<__nv_bfloat16, __nv_bfloat16, true>(p, tiles, tiles, gz, small, stream)
              : launch_grouped<__nv_bfloat16, __nv_bfloat16, false>(p, tiles, tiles, gz, small, stream);
  if (rc != LLMIE_OK) return rc;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
