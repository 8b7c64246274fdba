// Ring attention (context parallelism): the sequence is split over the ranks, every rank keeps
// its queries and the K/V blocks travel round the ring. ONE kernel per call does both halves:
//
//   communication CTAs (the first blockIdx values, so they are resident before anything spins):
//     step i = 0 .. W-2: take the block that originated on rank (r - i) - this rank's own K/V for
//     i = 0, else the copy that arrived in slot (r - i) of the local ring buffer, after waiting for
//     its arrival counter (acquire, bounded) - and forward it to slot (r - i) of rank r+1 with bulk
//     async copies HBM -> shared memory -> peer HBM, then raise that slot's counter on rank r+1
//     (release, system scope). Slots are indexed by origin rank, so nothing is overwritten inside
//     a call; across calls the buffer and counters are double-buffered by call parity.
//   attention CTAs (persistent): each takes (64-query tile, head) items and walks the blocks in
//     arrival order (own, r-1, r-2, ...), waiting for a block's counter only if it is not there yet;
//     flash-attention forward with online softmax on tensor cores (fp32 state in registers across
//     all blocks), K/V tiles streamed through a cp.async ring in swizzled shared memory.
//
// The reference has no ring attention (its only sequence-parallel path is the KV-split decode);
// causal masking assumes rank r holds tokens [r*S, (r+1)*S).
#include "ring_attention_common.cuh"

using namespace iris;

using namespace iris_ring;

namespace {

// ------------------------------------------------------------------ attention CTAs
template <bool kFp16>
__device__ void attn_main(const RingArgs& a, uint8_t* smem, int call) {
  const DeviceContext& ctx = a.ctx;
  const int W = ctx.world, r = ctx.rank;
  const int par = call & 1;
  const int32_t target = ((call >> 1) + 1) * a.n_comm;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = (a.S + kBQ - 1) / kBQ;
  const int items = q_tiles * a.Hq;
  const int group = a.Hq / a.Hkv;
  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
  const float scale2 = a.sm_scale * kLog2e;
  const size_t q_stride = (size_t)a.Hq * kD * 2, kv_stride = (size_t)a.Hkv * kD * 2;
  const size_t bb = block_bytes(a);
  __shared__ int s_ok;
  unsigned arrived_mask = 1u << r;    // blocks known to be present (own block always)

  for (int it = blockIdx.x - a.n_comm; it < items; it += gridDim.x - a.n_comm) {
    const int h = it % a.Hq, qt = it / a.Hq;
    const int kvh = h / group;
    const int q0 = qt * kBQ + warp * 16;     // first query row of this warp
    // Q fragments straight from global memory (rows q0 + lane/4 and +8)
    uint32_t qf[8][4];
    {
      const int r0 = q0 + (lane >> 2), r1 = r0 + 8, c0 = (lane & 3) * 2;
      const uint32_t* p0 = (const uint32_t*)(a.q + (size_t)r0 * q_stride + (size_t)h * kD * 2);
      const uint32_t* p1 = (const uint32_t*)(a.q + (size_t)r1 * q_stride + (size_t)h * kD * 2);
      const bool v0 = r0 < a.S, v1 = r1 < a.S;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int c = (ks * 16 + c0) >> 1;
        qf[ks][0] = v0 ? p0[c] : 0u; qf[ks][1] = v1 ? p1[c] : 0u;
        qf[ks][2] = v0 ? p0[c + 4] : 0u; qf[ks][3] = v1 ? p1[c + 4] : 0u;
      }
    }
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    for (int step = 0; step < W; ++step) {
      int origin = r - step;
      if (origin < 0) origin += W;
      if (a.causal && origin > r) continue;          // keys after all of my queries
      if (!((arrived_mask >> origin) & 1u)) {
        if (threadIdx.x == 0) s_ok = wait_flag_ge(ctx, a.flags + (size_t)par * W + origin, target) ? 1 : 0;
        __syncthreads();
        const bool ok = s_ok != 0;
        __syncthreads();
        if (!ok) return;
        arrived_mask |= 1u << origin;
      }
      const uint8_t* kb = origin == r ? a.k : slot_ptr(a, par, origin);
      const uint8_t* vb = origin == r ? a.v : slot_ptr(a, par, origin) + bb;
      const bool diag = a.causal && origin == r;
      // keys needed by this query tile: all of the block, or up to the tile's last row on the diagonal
      const int kv_end = diag ? min(a.S, qt * kBQ + kBQ) : a.S;
      const int n_tiles = (kv_end + kBKV - 1) / kBKV;
      auto issue_tile = [&](int t) {
        const int stage = t % kStages;
        const uint32_t ks = smem_base + stage * 2 * kTileBytes, vs = ks + kTileBytes;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int idx = threadIdx.x + i * kThreads;
          const int row = idx >> 4, chunk = idx & 15;
          const int pos = t * kBKV + row;
          if (pos < a.S) {
            const size_t e = (size_t)pos * kv_stride + (size_t)kvh * kD * 2 + chunk * 16;
            cp_async16(ks + tile_off(row, chunk), kb + e);
            cp_async16(vs + tile_off(row, chunk), vb + e);
          } else {
            *(uint4*)(smem + stage * 2 * kTileBytes + tile_off(row, chunk)) = make_uint4(0, 0, 0, 0);
            *(uint4*)(smem + stage * 2 * kTileBytes + kTileBytes + tile_off(row, chunk)) = make_uint4(0, 0, 0, 0);
          }
        }
      };
      __syncthreads();    // the previous block's last tile may still be read by another warp
      if (n_tiles > 0) issue_tile(0);
      cp_async_commit();
      for (int t = 0; t < n_tiles; ++t) {
        if (t + 1 < n_tiles) issue_tile(t + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int stage = t % kStages;
        const uint32_t ks = smem_base + stage * 2 * kTileBytes, vs = ks + kTileBytes;
        float s[8][4];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
          for (int np = 0; np < 4; ++np) {     // pairs of 8-key blocks
            uint32_t kf[4];
            const int j = lane >> 3, rr = lane & 7;
            ldsm4(kf, ks + tile_off(np * 16 + (j >> 1) * 8 + rr, kk * 2 + (j & 1)));
            mma<kFp16>(s[np * 2], qf[kk], kf[0], kf[1]);
            mma<kFp16>(s[np * 2 + 1], qf[kk], kf[2], kf[3]);
          }
        }
        // scale, mask, online softmax
        const int qrow0 = q0 + (lane >> 2), qrow1 = qrow0 + 8;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int pos = t * kBKV + nb * 8 + (lane & 3) * 2 + (e & 1);
            const int qr = (e >> 1) ? qrow1 : qrow0;
            float v = s[nb][e] * scale2;
            if (pos >= a.S || (diag && pos > qr)) v = -INFINITY;
            s[nb][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
          }
        float alpha[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          mx[q] = fmaxf(mx[q], __shfl_xor_sync(0xffffffffu, mx[q], 1));
          mx[q] = fmaxf(mx[q], __shfl_xor_sync(0xffffffffu, mx[q], 2));
          const float m_new = fmaxf(m_run[q], mx[q]);
          alpha[q] = m_new == -INFINITY ? 1.f : exp2f(m_run[q] - m_new);
          m_run[q] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        uint32_t pf[4][4];      // P as A operand: 4 k-steps of 16 keys
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
          float p[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float mr = m_run[e >> 1];
            p[e] = mr == -INFINITY ? 0.f : exp2f(s[nb][e] - mr);
            rs[e >> 1] += p[e];
          }
          pf[nb >> 1][(nb & 1) * 2 + 0] = pack2<kFp16>(p[0], p[1]);
          pf[nb >> 1][(nb & 1) * 2 + 1] = pack2<kFp16>(p[2], p[3]);
        }
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          rs[q] += __shfl_xor_sync(0xffffffffu, rs[q], 1);
          rs[q] += __shfl_xor_sync(0xffffffffu, rs[q], 2);
          l_run[q] = l_run[q] * alpha[q] + rs[q];
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
          o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {       // 16 keys per k-step
#pragma unroll
          for (int nb2 = 0; nb2 < 8; ++nb2) {
            uint32_t vf[4];
            const int j = lane >> 3, rr = lane & 7;
            ldsm4t(vf, vs + tile_off(kk * 16 + (j & 1) * 8 + rr, nb2 * 2 + (j >> 1)));
            mma<kFp16>(o[nb2 * 2], pf[kk], vf[0], vf[1]);
            mma<kFp16>(o[nb2 * 2 + 1], pf[kk], vf[2], vf[3]);
          }
        }
        __syncthreads();
      }
      cp_async_wait<0>();
    }
    // write the item: rows q0 + lane/4 (+8), columns i*8 + (lane%4)*2
    {
      const int r0 = q0 + (lane >> 2), r1 = r0 + 8, c0 = (lane & 3) * 2;
      const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (r0 < a.S) *(uint32_t*)(a.out + (size_t)r0 * q_stride + ((size_t)h * kD + i * 8 + c0) * 2) = pack2<kFp16>(o[i][0] * inv0, o[i][1] * inv0);
        if (r1 < a.S) *(uint32_t*)(a.out + (size_t)r1 * q_stride + ((size_t)h * kD + i * 8 + c0) * 2) = pack2<kFp16>(o[i][2] * inv1, o[i][3] * inv1);
      }
      if (a.lse && (lane & 3) == 0) {
        if (r0 < a.S) a.lse[(size_t)r0 * a.Hq + h] = l_run[0] > 0.f ? (m_run[0] + log2f(l_run[0])) / kLog2e : -INFINITY;
        if (r1 < a.S) a.lse[(size_t)r1 * a.Hq + h] = l_run[1] > 0.f ? (m_run[1] + log2f(l_run[1])) / kLog2e : -INFINITY;
      }
    }
  }
}

template <bool kFp16>
__global__ void __launch_bounds__(kThreads) ring_attention_kernel(const __grid_constant__ RingArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int call = *(volatile int32_t*)&a.state[0];
  if ((int)blockIdx.x < a.n_comm) comm_main(a, smem, kStages * 2 * kTileBytes, call);
  else attn_main<kFp16>(a, smem, call);
  finish_call(a, call);
}

}  // namespace

extern "C" {

typedef struct IrisRingAttnDesc {
  IrisCtx ctx;
  const void* q; const void* k; const void* v;
  void* kv_buf; int32_t* flags; int32_t* state;
  void* out; float* lse;
  int32_t S, Hq, Hkv, D, causal, n_comm, dtype;
  int32_t options;        // bit 0: use the mma.sync attention CTAs; bit 1: zigzag layout (needs S % 256 == 0)
  float sm_scale;
} IrisRingAttnDesc;

// Bytes of heap the ring buffer needs: [2][W][2][S, Hkv, D] 16-bit.
unsigned long long iris_ring_attention_workspace(int W, int S, int Hkv, int D) {
  return 2ull * W * 2ull * S * Hkv * D * 2ull;
}

int iris_ring_attention(const IrisRingAttnDesc* d, void* stream) {
  if (d->D != kD || d->Hq % d->Hkv) return -3;
  if (d->dtype != IRIS_BF16 && d->dtype != IRIS_F16) return -2;
  if (d->ctx.world > 32) return -4;
  RingArgs a;
  memcpy(&a.ctx, &d->ctx, sizeof(DeviceContext));
  a.q = (const uint8_t*)d->q; a.k = (const uint8_t*)d->k; a.v = (const uint8_t*)d->v;
  a.kv_buf = (uint8_t*)d->kv_buf; a.flags = d->flags; a.state = d->state;
  a.out = (uint8_t*)d->out; a.lse = d->lse;
  a.S = d->S; a.Hq = d->Hq; a.Hkv = d->Hkv; a.causal = d->causal; a.is_fp16 = d->dtype == IRIS_F16;
  a.n_comm = d->ctx.world > 1 ? (d->n_comm > 0 ? d->n_comm : 8) : 0;
  a.sm_scale = d->sm_scale;
  a.zigzag = (d->options & 2) ? 1 : 0;
  if (a.zigzag && (d->S % 256 || (d->options & 1))) return -3;     // only the tcgen05 CTAs know the zigzag layout
  if (!(d->options & 1)) {
    const int r = launch_ring_attention_tc(a, (cudaStream_t)stream);
    if (r <= 0) return r;
    if (a.zigzag) return -3;
  }
  const int smem = kStages * 2 * kTileBytes;   // 64 KB: three CTAs per SM
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(ring_attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -20;
    if (cudaFuncSetAttribute(ring_attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -20;
    attr = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int items = ((d->S + kBQ - 1) / kBQ) * d->Hq;
  int attn = items < 2 * sms ? items : 2 * sms;   // resident: waits never starve the comm CTAs
  if (attn < 1) attn = 1;
  const int grid = a.n_comm + attn;
  if (a.is_fp16) ring_attention_kernel<true><<<grid, kThreads, smem, (cudaStream_t)stream>>>(a);
  else ring_attention_kernel<false><<<grid, kThreads, smem, (cudaStream_t)stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // extern "C"
