// Split-KV across GPUs: exchange of the ranks' partial results and their LSE-combine in ONE kernel over peer memory.
//
// Every rank has decoded its slice of the keys to a partial (O fp32 normalised by its own softmax sum, natural-log LSE)
// per (sequence, head, token) row.  Each rank owns an exchange buffer that all other ranks have mapped (CUDA IPC); a
// launch of this kernel on rank r, one CTA per row,
//   1. stores the row's partial into slot r of EVERY rank's buffer (plain stores, over NVLink for the peers), makes
//      them visible system-wide and then sets that row's flag of slot r in the same buffer to the call's epoch;
//   2. waits (bounded) until the flags of all slots of its OWN buffer show the epoch, i.e. until every rank's partial
//      of this row has arrived;
//   3. combines the row over the slots exactly as combine_kernel does and writes the final output.
// There is no grid-wide step: rows are independent, a row's 129 floats per rank travel as soon as its CTA runs.
// The buffer is double: calls alternate between its halves by the parity of the epoch.  A rank can run at most one
// call ahead of the slowest one (its next call waits for that rank's flags, which are set by a kernel that follows the
// reading one in that rank's stream), so a half is never overwritten while somebody still reads it.
// Replaces all_gather + combine of the reference-style split (three launches and a collective per step) by one launch.
#include "fa_common.cuh"
#include "fa_kernels.h"

namespace fa {

size_t exchange_region_bytes(int world, int rows, int d) {
  const size_t raw = static_cast<size_t>(world) * rows * (static_cast<size_t>(d) + 2) * 4;
  return (raw + 255) & ~static_cast<size_t>(255);
}

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

constexpr int kExchangeThreads = 128;

__global__ void __launch_bounds__(kExchangeThreads) exchange_combine_kernel(const ExchangeKernelParams p) {
  __shared__ float sm_lse[kMaxExchangeRanks];
  __shared__ volatile int sm_abort;
  const int row = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nv = p.d >> 2;   // float4 pieces of a row
  const size_t slots = static_cast<size_t>(p.world) * p.rows;
  const size_t o_off = (p.epoch & 1u) * p.region_bytes;
  const size_t l_off = o_off + slots * p.d * 4;
  const size_t f_off = l_off + slots * 4;
  const size_t my_slot = static_cast<size_t>(p.rank) * p.rows + row;
  if (tid == 0) sm_abort = 0;

  // Launched with programmatic stream serialisation: the CTAs may be resident before the decode kernel that produces
  // o_local / lse_local has finished; nothing above touched global memory.
  griddep_wait();
  if (p.do_push) {
    const float4* src = reinterpret_cast<const float4*>(p.o_local) + static_cast<size_t>(row) * nv;
    const float my_lse = p.lse_local[row];
    // each warp serves the ranks warp, warp + 4, ...: first all its stores, one system-wide fence for them together
    // (a fence waits for the peers' acknowledgements, a round trip over NVLink), then the flags
    for (int dst = warp; dst < p.world; dst += kExchangeThreads / 32) {
      uint8_t* base = static_cast<uint8_t*>(p.peers[dst]);
      float4* od = reinterpret_cast<float4*>(base + o_off) + my_slot * nv;
      for (int c = lane; c < nv; c += 32) od[c] = src[c];
      if (lane == 0) reinterpret_cast<float*>(base + l_off)[my_slot] = my_lse;
    }
    __threadfence_system();
    __syncwarp();
    if (lane == 0)
      for (int dst = warp; dst < p.world; dst += kExchangeThreads / 32)
        st_release_sys(reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(p.peers[dst]) + f_off) + my_slot, p.epoch);
  }
  __syncthreads();

  uint8_t* mine = static_cast<uint8_t*>(p.peers[p.rank]);
  if (p.do_wait && tid < p.world) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + f_off) + static_cast<size_t>(tid) * p.rows + row;
    long long t0 = 0;
    uint32_t it = 0;
    while (ld_acquire_sys(flag) != p.epoch) {
      if ((++it & 63u) == 0u) {
        const long long now = clock64();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > kWaitLimitCycles || sm_abort) {
          if (!sm_abort) atomicOr(p.status, FA_B200_ERR_DEVICE_TIMEOUT);
          sm_abort = 1;
          break;
        }
      }
    }
  }
  __syncthreads();
  if (sm_abort) return;

  // ---- combine the row over the ranks' slots (same arithmetic as combine_kernel)
  if (tid < p.world) {
    float l = __ldcg(reinterpret_cast<const float*>(mine + l_off) + static_cast<size_t>(tid) * p.rows + row);
    if (l == INFINITY) l = -INFINITY;
    sm_lse[tid] = l;
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int i = 0; i < p.world; ++i) mx = fmaxf(mx, sm_lse[i]);
  float sum = 0.f;
  if (mx != -INFINITY)
    for (int i = 0; i < p.world; ++i) sum += expf(sm_lse[i] - mx);
  const int sq = p.sq > 0 ? p.sq : 1;
  const int bi = row / (p.h * sq), hi = (row / sq) % p.h, ti = row % sq;
  if (p.s_aux) {   // the attention sink of this head: one more term e^sink of the row's sum
    const float sink = load_sink_log2(p.s_aux, p.s_aux_dtype, hi) * kLn2;
    const float m2 = fmaxf(mx, sink);
    sum = (mx == -INFINITY ? 0.f : sum * expf(mx - m2)) + expf(sink - m2);
    mx = m2;
  }
  const bool empty = !(sum > 0.f);
  const float lse_tot = empty ? 0.f : mx + logf(sum);
  for (int c = tid; c < nv; c += kExchangeThreads) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!empty) {
      for (int i = 0; i < p.world; ++i) {   // fixed order: the result does not depend on arrival order
        const float l = sm_lse[i];
        const float w = (l == -INFINITY) ? 0.f : expf(l - lse_tot);
        if (w != 0.f) {   // a weight of exactly zero must not pick up NaN/Inf from an unused partial
          const float4 v = __ldcg(reinterpret_cast<const float4*>(mine + o_off) + (static_cast<size_t>(i) * p.rows + row) * nv + c);
          a.x += w * v.x; a.y += w * v.y; a.z += w * v.z; a.w += w * v.w;
        }
      }
    }
    if (p.out) {
      const int64_t off = static_cast<int64_t>(bi) * p.out_batch_stride + static_cast<int64_t>(hi) * p.out_row_stride +
                          static_cast<int64_t>(ti) * p.out_tok_stride + 4 * c;
      if (p.out_dtype == FA_B200_BF16) {
        __nv_bfloat162 x = __floats2bfloat162_rn(a.x, a.y), y = __floats2bfloat162_rn(a.z, a.w);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off) =
            make_uint2(*reinterpret_cast<uint32_t*>(&x), *reinterpret_cast<uint32_t*>(&y));
      } else if (p.out_dtype == FA_B200_F16) {
        __half2 x = __floats2half2_rn(a.x, a.y), y = __floats2half2_rn(a.z, a.w);
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.out) + off) =
            make_uint2(*reinterpret_cast<uint32_t*>(&x), *reinterpret_cast<uint32_t*>(&y));
      } else {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + off) = a;
      }
    }
  }
  if (p.lse && tid == 0) p.lse[row] = empty ? INFINITY : lse_tot;
}

}  // namespace

cudaError_t launch_exchange_combine(const ExchangeKernelParams& p, cudaStream_t stream) {
  if (p.rows <= 0) return cudaSuccess;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.rows);
  cfg.blockDim = dim3(kExchangeThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.dependent_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, exchange_combine_kernel, p);
}

}  // namespace fa
