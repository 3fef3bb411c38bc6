// Sender role of the fused expert-parallel kernel: a few CTAs of the persistent GEMM grid do
// not multiply but push this rank's token rows to the ranks that own their experts, phase by
// phase (phase p -> rank + p), while the other CTAs multiply the rows that have already arrived.
//
// A sender CTA moves rows global -> shared with bulk async copies (cp.async.bulk, completion on an
// mbarrier: one thread keeps several KB in flight per warp without registers) and shared -> peer
// memory with plain 16-byte stores (posted writes over NVLink).  Every warp works on its own:
// own slots, own barriers, its share of the phase's rows (taken from the send list the assign
// kernel wrote), so there is no hand-over between warps.  The copying warps never fence: when
// one has issued all its stores of a phase it arrives on that phase's CTA barrier and goes on
// with the next phase.  Warp 0 of the CTA copies nothing; per phase it waits for the others'
// arrivals, fences at system scope (the fence is cumulative: it covers the stores of the warps
// whose arrival it has observed) and counts the CTA in; the last CTA stores the epoch into the
// destination's ready flag for this source, which is what the destination's GEMM loader waits
// for (wait_flag_ge).
//
// Only local memory is read by the bulk copies; peer memory is only written, with plain stores.
#pragma once

#include <stdint.h>

#include "rd_ptx.cuh"

namespace rd {

constexpr int kEpChunkBytes = 4096;  // bytes per bulk copy / slot
constexpr int kEpSlots = 4;          // slots per warp: three copies in flight while one is stored

struct EpSendArgs {
  const uint8_t* x;           // [tokens, row_bytes] rows to send
  const int32_t* send_index;  // (token, slot) entries grouped by phase
  const int32_t* send_start;  // [world + 1] first list position of each phase
  const int32_t* dest_pos;    // [tokens * top_k] row position at the owner (-1: dropped)
  int32_t* phase_done;        // [world] warps that have finished a phase (reset by the plan)
  const uint64_t* peer_base;   // [world] device array: receive buffer of rank r as seen from this GPU
  const uint64_t* peer_flags;  // [world] device array: ready-flag array of rank r as seen from this GPU
  int row_bytes, top_k, world, rank, capacity_rows, sender_ctas;  // world == 0: no sender role
};

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// Runs on every thread of a sender CTA.  smem: 1024-byte aligned shared window of at least
// warps * (kEpSlots * kEpChunkBytes + 64) + 8 * world bytes.
__device__ __noinline__ void ep_sender_role(const EpSendArgs a, int epoch, int sender, uint32_t smem,
                                            volatile WaitCtl* abort_flag, uint32_t wait_limit_us,
                                            int32_t* status) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_warps = blockDim.x >> 5;
  const uint64_t t_start = global_timer_ns();
  if (threadIdx.x == 0) {
    abort_flag->abort = 0;
    abort_flag->limit_us = wait_limit_us;
  }
  const uint32_t slots = smem + warp * (kEpSlots * kEpChunkBytes);
  const uint32_t bars = smem + n_warps * (kEpSlots * kEpChunkBytes) + warp * 64;
  const uint32_t phase_bars = smem + n_warps * (kEpSlots * kEpChunkBytes + 64);  // one per phase
  if (lane == 0) {
    for (int s = 0; s < kEpSlots; ++s) mbar_init(bars + 8 * s, 1);
    if (warp == 0)
      for (int p = 0; p < a.world; ++p) mbar_init(phase_bars + 8 * p, n_warps - 1);
    fence_mbar_init();
  }
  __syncthreads();

  const int cpr = (a.row_bytes + kEpChunkBytes - 1) / kEpChunkBytes;  // chunks per row
  const int n_copy = n_warps - 1;                                        // warp 0 only signals
  const long long GW = static_cast<long long>(a.sender_ctas) * n_copy;  // warps copying
  const long long gw = static_cast<long long>(sender) * n_copy + (warp - 1);
  uint32_t parity = 0;  // bit s: parity of the next completion of slot s
  bool ok = true;

  if (warp == 0) {
    // ---- signaller
    for (int p = 1; p < a.world && ok; ++p) {
      if (!mbar_wait(phase_bars + 8 * p, 0u, abort_flag)) {
        ok = false;
        break;
      }
      __threadfence_system();
      if (lane == 0) {
        const int dest = (a.rank + p) % a.world;
        const int done = atomicAdd(a.phase_done + p, 1) + 1;
        if (done == a.sender_ctas) {
          __threadfence_system();
          int32_t* flag = reinterpret_cast<int32_t*>(a.peer_flags[dest]) + p;
          asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
        }
      }
      __syncwarp();
    }
  }
  for (int p = 1; warp > 0 && p < a.world && ok; ++p) {
    const int dest = (a.rank + p) % a.world;
    uint8_t* dst_base = reinterpret_cast<uint8_t*>(a.peer_base[dest]);
    const int start = a.send_start[p];
    const long long units = static_cast<long long>(a.send_start[p + 1] - start) * cpr;
    const int n = gw < units ? static_cast<int>((units - gw + GW - 1) / GW) : 0;  // this warp's units

    // Unit t of this warp is global unit gw + t * GW = (list entry, chunk).  Lane l holds the
    // description of unit 32 * batch + l; two batches are kept so copies can run ahead.
    long long src_c = 0, dst_c = 0, src_n = 0, dst_n = 0;
    int bytes_c = 0, bytes_n = 0;
    auto describe = [&](int batch, long long& src, long long& dst, int& bytes) {
      src = dst = 0;
      bytes = 0;
      const long long t = static_cast<long long>(batch) * 32 + lane;
      if (t >= n) return;
      const long long u = gw + t * GW;
      const int entry = a.send_index[start + static_cast<int>(u / cpr)];
      const int chunk = static_cast<int>(u % cpr);
      const int pos = a.dest_pos[entry];
      if (pos < 0 || pos >= a.capacity_rows) return;
      const int off = chunk * kEpChunkBytes;
      src = static_cast<long long>(entry / a.top_k) * a.row_bytes + off;
      dst = static_cast<long long>(pos) * a.row_bytes + off;
      bytes = a.row_bytes - off < kEpChunkBytes ? a.row_bytes - off : kEpChunkBytes;
    };
    describe(0, src_c, dst_c, bytes_c);
    describe(1, src_n, dst_n, bytes_n);

    int issued = 0;
    for (int t = 0; t < n && ok; ++t) {
      if (t > 0 && (t & 31) == 0) {  // entering the next batch
        src_c = src_n;
        dst_c = dst_n;
        bytes_c = bytes_n;
        describe((t >> 5) + 1, src_n, dst_n, bytes_n);
      }
      const int cur_batch = t >> 5;
      // Start the copies of the next units: up to kEpSlots - 1 ahead of the one stored now.
      // Unit `issued` reuses the slot of unit issued - kEpSlots <= t - 1, whose stores have all
      // been issued (and their shared-memory reads done) before the __syncwarp below.
      while (issued < n && issued < t + kEpSlots) {
        const bool in_cur = (issued >> 5) == cur_batch;
        const long long s = __shfl_sync(0xffffffffu, in_cur ? src_c : src_n, issued & 31);
        const int by = __shfl_sync(0xffffffffu, in_cur ? bytes_c : bytes_n, issued & 31);
        if (by > 0 && lane == 0) {
          const int slot = issued % kEpSlots;
          mbar_arrive_expect_tx(bars + 8 * slot, by);
          bulk_load_1d(slots + slot * kEpChunkBytes, a.x + s, by, bars + 8 * slot);
        }
        ++issued;
      }
      const long long d = __shfl_sync(0xffffffffu, dst_c, t & 31);
      const int by = __shfl_sync(0xffffffffu, bytes_c, t & 31);
      if (by > 0) {
        const int slot = t % kEpSlots;
        if (!mbar_wait(bars + 8 * slot, (parity >> slot) & 1u, abort_flag)) {
          ok = false;
          break;
        }
        parity ^= 1u << slot;
        const uint32_t sbase = slots + slot * kEpChunkBytes;
        uint8_t* dptr = dst_base + d;
        for (int off = lane * 16; off < by; off += 512) {
          uint4 v;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                       : "r"(sbase + off)
                       : "memory");
          *reinterpret_cast<uint4*>(dptr + off) = v;
        }
      }
      __syncwarp();
    }
    if (!ok) break;
    // This warp's stores of phase p have been issued: tell the signaller and go on.
    __syncwarp();
    if (lane == 0) mbar_arrive(phase_bars + 8 * p);
    __syncwarp();
  }

  __syncthreads();
  // status[1]: time the slowest sender CTA needed for all its phases (microseconds)
  if (threadIdx.x == 0)
    atomicMax(status + 1, static_cast<int32_t>((global_timer_ns() - t_start) / 1000ull));
  if (abort_flag->abort) {
    if (threadIdx.x == 0) atomicMax(status, 1);
    // bulk copies may still be in flight into this CTA's shared memory
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
}

}  // namespace rd
