// Parameter block of the masked-attention kernels (shared by the launchers and the
// torch bindings).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb200 {

struct AttnParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* ke;
  const __nv_bfloat16* ve;
  const int* lo;
  const int* hi;
  const int* ext_idx;
  __nv_bfloat16* out;
  float* lse2;  // [nh, Tq] log2-domain logsumexp of the scaled scores
  int Tq, Tc, Te, E, nh, nkv;
  // Block-structured extra keys (tcgen05 kernels): when ext_block = B > 0 the extra keys of query row r are
  // the rows [B * (r / B), B * (r / B) + B) of the extra K / V tensors (only up to r itself with ext_causal):
  // the anchored blocks of DFlash / DSpark, whose 16 block keys are shared by the 16 rows of a block.  The 128
  // extra rows that belong to a 128-row query tile then form one more key tile with a block-diagonal mask and
  // go through the tensor-core path like any context tile; ext_idx is not read (E must be 0).
  int ext_block, ext_causal;
  int64_t q_rs, k_rs, v_rs, ke_rs, ve_rs, o_rs;
  float scale;
  // backward only
  const __nv_bfloat16* dout;
  int64_t do_rs;
  float* delta;          // [nh, Tq]
  __nv_bfloat16* dq;     // [Tq, nh, HD] row stride dq_rs
  int64_t dq_rs;
  float* dke;            // [Te, nkv, HD] fp32 (atomics)
  float* dve;
  __nv_bfloat16* dk;     // [Tc, nkv, HD] contiguous
  __nv_bfloat16* dv;
  float* dkv_part;       // [group, 2, Tc, nkv, HD] fp32 per-query-head partials of dK / dV (grouped-query attention only)
  const int* tile_qmin;  // [ceil(Tc / kBN)] first / one-past-last query row that can see the kv tile
  const int* tile_qmax;
};

int launch_attn_fwd(const AttnParams& p, int hd, cudaStream_t stream);
// tcgen05 forward, head_dim 128; `status`: device int that receives a code when a bounded wait expires.
int launch_attn_fwd_tc(const AttnParams& p, int* status, cudaStream_t stream);
// tile_qmin / tile_qmax: scratch of one int per 64-key tile, fully written by the launch.
int launch_attn_bwd(const AttnParams& p, int hd, int* tile_qmin, int* tile_qmax, cudaStream_t stream);
constexpr int kAttnKeyTile = 64;
// tcgen05 backward (dQ kernel, dK/dV kernel), head_dim 128; same scratch and status conventions.
int launch_attn_bwd_tc(const AttnParams& p, int* tile_qmin, int* tile_qmax, int* status, cudaStream_t stream);
// Pieces of the backward shared by both implementations: per-64-key-tile query row ranges,
// and the head-ordered sum of the fp32 dK / dV partials of grouped queries (head_dim 128).
int launch_kv_tile_range(const AttnParams& p, int* tile_qmin, int* tile_qmax, cudaStream_t stream);
int launch_dkv_reduce(const AttnParams& p, cudaStream_t stream);

}  // namespace sb200
