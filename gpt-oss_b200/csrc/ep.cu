// Expert parallelism: dispatch -> owner experts -> return -> combine.
//
// Replaces gpu_forward_device_batch_ep and run_owner_mlp of the reference
// (getp-csrc/expert.cpp:1366-1607, :175-437), its per-owner routing / packing
// kernels (getp-csrc/utility/utility.cpp:830-1016) and the host rendezvous
// (expert.cpp:67-173).  Kept from the reference: owner of expert e is rank
// e % N with local id e / N; a token's row travels once to an owner even when
// several of its experts live there.  Not kept: host mutexes, one routing launch
// per owner, per-(home, expert) copy loops and memsets.
//
// Every rank is a home (its own tokens) and an owner (E / N experts).  Two transports.
//
// Peer memory ("ep_transport" 1, the default wherever the ranks can address each
// other's buffers): no row is packed, sent or received, and the layer makes no NCCL
// call and no host synchronisation.  Every rank keeps its activations in a buffer its
// peers can read and writes its routing result (expert ids and weights of its tokens,
// a few hundred KB) straight into every peer's memory, followed by a flag (release
// store at system scope, after the kernel that wrote the data has ended).  Each
// owner waits for the N flags (acquire polls with a time limit), sorts ALL tokens
// of all ranks by its local experts, and its gather kernel pulls the rows it needs
// out of the home ranks' memory over NVLink into expert order - dispatch and gather
// are one kernel; a token with several experts on this owner crosses the link once.  The owner's down GEMM then stores every weighted expert output row
// straight into the memory of the rank its token came from (slot (t, k) of that rank's
// receive buffer; the destination of each sorted row is worked out once per layer), so the
// return trip runs under the GEMM's own tiles: the bulk stores of its epilogue cross
// NVLink while the tensor cores work on the next tile.  A second round of flags says
// "expert outputs delivered", and the home's combine kernel waits for them and adds the
// token's K rows from its own memory, in slot order in fp32, and the residual - the sum is
// the single-GPU combine's, the same K rows in the same order: sharding adds no rounding
// of its own.  ("ep_push" 0 keeps the outputs at the owner and lets the home's combine
// kernel fetch them over NVLink after the flags, the position from the owner's inverse
// permutation: the same sum, 0.1-0.2 ms more per layer.  The reference's owner first sums
// its experts' outputs per row and rounds that to bf16, expert.cpp:394-410: one more
// rounding per owner and one more pass over the outputs, for a little less traffic.)
// A rank reuses a buffer only after the flags that prove its readers or writers are done:
// activations and routing slots after the second flags of the same layer (every peer has
// gathered), its receive buffer is written again only after the first flags of the next
// layer (this rank has combined before it published).
//
// NCCL send / recv ("ep_transport" 0, the fallback, one process per rank), per layer:
//   1. home: mark for every token the owners it needs; counting sort of the
//      (token, owner) pairs by owner with the permutation kernels -> per-owner
//      send lists in token order; pack rows and per-row slot metadata
//   2. counts: all-gather of the N send counts, one small D2H copy and the only
//      host synchronisation of the layer (NCCL point-to-point sizes are host
//      arguments)
//   3. dispatch: grouped ncclSend / ncclRecv; received rows land in this rank's
//      own HBM before any kernel or TMA touches them
//   4. owner: the single-GPU expert stage on the received rows, then the owner sums
//      its experts' weighted outputs per received row in fp32 and rounds to bf16
//      (the reference's pre-reduction)
//   5. return: grouped send / recv the other way
//   6. home: x += sum over owners of the returned rows (the combine kernel with
//      one slot per owner)
// Ranks must call the layer in lock step (also with zero tokens).
//
// The peer-memory transport has two ways to learn the peers' addresses: CUDA IPC handles
// exchanged over the NCCL communicator (one process per rank, gptoss_moe_ep_init), or
// plain pointers when one process drives all GPUs with a host thread each, as the
// reference's getp engine does (gptoss_moe_ep_init_local: peer access enabled between
// the devices, no NCCL, no IPC).
//
// NCCL is loaded with dlopen on first use, so single-GPU users of the library do
// not need it; in a process that already loaded NCCL (PyTorch) the same copy is
// picked up.
#include "ep.h"

#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <unistd.h>

#include <vector>

#include "common.cuh"

namespace gptoss {

struct NcclApi {
  void *lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi g_nccl;

static bool load_nccl(std::string *err) {
  if (g_nccl.lib) return true;
  void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) {
    *err = std::string("cannot load NCCL: ") + dlerror();
    return false;
  }
#define SYM(field, name)                                                  \
  *reinterpret_cast<void **>(&g_nccl.field) = dlsym(lib, name);           \
  if (!g_nccl.field) {                                                    \
    *err = std::string("NCCL symbol missing: ") + name;                   \
    return false;                                                         \
  }
  SYM(GetUniqueId, "ncclGetUniqueId")
  SYM(CommInitRank, "ncclCommInitRank")
  SYM(CommDestroy, "ncclCommDestroy")
  SYM(Send, "ncclSend")
  SYM(Recv, "ncclRecv")
  SYM(AllGather, "ncclAllGather")
  SYM(GroupStart, "ncclGroupStart")
  SYM(GroupEnd, "ncclGroupEnd")
  SYM(GetErrorString, "ncclGetErrorString")
#undef SYM
  g_nccl.lib = lib;
  return true;
}

struct EpState {
  ncclComm_t comm = nullptr;
  int N = 1, rank = 0;
  int send_cap = 0;  // rows this rank can send: T * min(N, K)
  // home side: (token, owner) plan
  int *own_key = nullptr;       // [T, N] owner id or -1
  float *own_w = nullptr;       // [T, N] unused weights (zeros)
  int *s_block_counts = nullptr, *s_offsets = nullptr, *s_sorted_row = nullptr;
  float *s_sorted_w = nullptr;
  int *s_row_of = nullptr;
  int *s_mtile = nullptr;       // dummy tile schedule (3 arrays + count)
  int s_mtiles_cap = 0, s_blocks_cap = 0;
  bf16 *send_rows = nullptr;    // [send_cap, H]
  int *send_e = nullptr;        // [send_cap, K] local expert id at the owner or -1
  float *send_w = nullptr;      // [send_cap, K]
  bf16 *ret_rows = nullptr;     // [send_cap, H] partial sums coming back
  // owner side
  bf16 *recv_rows = nullptr;    // [N*T, H]
  int *recv_e = nullptr;        // [N*T, K]
  float *recv_w = nullptr;      // [N*T, K]
  bf16 *out_rows = nullptr;     // [N*T, H] per-row sums over this rank's experts (NCCL transport)
  int *counts_dev = nullptr;    // [N, N] counts_dev[src][dst]
  int *counts_host = nullptr;   // pinned copy
  // peer-memory transport
  int transport = 0;            // 0 = NCCL send / recv, 1 = peer loads
  bool peer_ok = false;
  bool local = false;           // peers wired inside one process (no IPC mappings to close)
  std::string peer_why;         // why the peer transport is not available
  int max_t = 0;
  bf16 *pub_t = nullptr;        // [max_t, H] this rank's activations, mapped by the peers
  int *ctl = nullptr;           // mapped by the peers: flags [2][N], then all_meta
  int *all_meta = nullptr;      // ctl + kCtlHeader: [N][2 * max_t * K] expert ids, then weights
  void *peer_ctl[GPTOSS_MAX_TOPK] = {};  // peers' ctl (own entry: the local buffer)
  cudaStream_t s2 = nullptr;    // second stream: the gather of the second half of the experts
  cudaEvent_t ev_plan = nullptr, ev_second = nullptr;
  int round = 0;
  void *peer_t[GPTOSS_MAX_TOPK] = {};    // peers' pub_t (own entry: the local buffer)
  void *peer_out[GPTOSS_MAX_TOPK] = {};    // peers' expert outputs (their engine's ys)
  void *peer_rowof[GPTOSS_MAX_TOPK] = {};  // peers' inverse permutation (their engine's row_of)
  bf16 *recv_out = nullptr;                // [max_t * K, H] expert outputs of this rank's tokens,
                                           // stored here by the owners' down GEMMs (ep_push)
  void *peer_recv[GPTOSS_MAX_TOPK] = {};   // peers' recv_out (own entry: the local buffer)
};

struct PeerRows {
  const bf16 *p[GPTOSS_MAX_TOPK];
};
struct PeerCtl {
  int *p[GPTOSS_MAX_TOPK];
};
struct PeerInts {
  const int *p[GPTOSS_MAX_TOPK];
};
constexpr int kCtlHeader = 64;  // ints in front of all_meta: flags[which][source rank]

// flags[which][rank] = round in every peer's control block.  Launched after the kernel
// that produced the data the flag announces: that kernel has ended, so its writes (to
// this GPU's memory or to the peers') are done before these stores are issued.
__global__ void ep_signal_kernel(const PeerCtl ctl, int N, int which, int rank, int round) {
  const int p = threadIdx.x;
  if (p >= N) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(ctl.p[p] + which * N + rank), "r"(round)
               : "memory");
}

// Waits until every rank's flag of this round is here; false (and a status) after
// kWaitLimitNs.  Called by the first warp of a CTA, followed by a CTA barrier.
__device__ __forceinline__ bool ep_wait_flags(const int *flags, int N, int round, int *status,
                                              uint64_t limit_ns) {
  const int lane = threadIdx.x & 31;
  bool ok = true;
  if (lane < N) {
    const int *f = flags + lane;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
      int v;
      asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (v - round >= 0) break;
      if ((++spins & 0xff) == 0) {
        const uint64_t now = global_timer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > limit_ns) {
          set_status(status, kStatusWaitTimeoutPeer);
          ok = false;
          break;
        }
      }
    }
  }
  return __all_sync(0xffffffffu, ok);
}

// This rank's routing result, written into slot `rank` of all_meta in every rank's
// control block (its own included): ids of rows >= T are -1.
__global__ void __launch_bounds__(256)
ep_publish_meta_kernel(const int *__restrict__ topk_i, const float *__restrict__ topk_v, int T,
                       int max_t, int K, const PeerCtl ctl, int N, int rank) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int per = max_t * K;
  if (i >= per) return;
  const bool live = i < T * K;
  const int id = live ? topk_i[i] : -1;
  const int w = live ? __float_as_int(topk_v[i]) : 0;
  const size_t off = kCtlHeader + static_cast<size_t>(rank) * 2 * per + i;
#pragma unroll
  for (int p = 0; p < GPTOSS_MAX_TOPK; p++) {
    if (p < N) {
      ctl.p[p][off] = id;
      ctl.p[p][off + per] = w;
    }
  }
}

// Owner view of every rank's tokens: global row g = src * max_t + t keeps the slots
// whose expert lives here (local id e / N), the others become -1.
__global__ void __launch_bounds__(256)
ep_owner_slots_kernel(const int *all_meta, const int *flags, int round, int N, int rank,
                      int max_t, int K, int *__restrict__ stage_e, float *__restrict__ stage_w,
                      int *status, uint64_t limit_ns) {
  // every rank's routing result (and, by the order of its stream, its activations)
  if (threadIdx.x < 32) ep_wait_flags(flags, N, round, status, limit_ns);
  __syncthreads();
  const int per = max_t * K;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * per) return;
  const int src = i / per, j = i - src * per;
  const int e = all_meta[static_cast<size_t>(src) * 2 * per + j];
  const bool mine = e >= 0 && e % N == rank;
  stage_e[i] = mine ? e / N : -1;
  stage_w[i] = mine ? __int_as_float(all_meta[static_cast<size_t>(src) * 2 * per + per + j]) : 0.f;
}

struct PeerBytes {
  unsigned long long p[GPTOSS_MAX_TOPK];
};

// row_dst[pos] = where the expert output of sorted row pos belongs: slot (t, k) of the receive
// buffer of the rank the token came from.  One thread per (global row, slot).
__global__ void __launch_bounds__(256)
ep_row_dst_kernel(const int *__restrict__ row_of, const PeerBytes recv, int N, int per, int H,
                  int assign_cap, unsigned long long *__restrict__ row_dst) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * per) return;
  const int pos = row_of[i];
  if (pos < 0 || pos >= assign_cap) return;
  const int src = i / per, j = i - src * per;  // j = t * K + k at the home rank
  row_dst[pos] = recv.p[src] + static_cast<unsigned long long>(j) * H * sizeof(bf16);
}

// xs[r, :] = activations of global row sorted_row[r], read from the home rank's
// published buffer (a peer mapping for every rank but this one); one warp per row,
// eight 16-byte loads in flight per lane to cover the NVLink round trip.
// A token that has several of its experts on this rank crosses the link once: pass 0
// fetches, of a remote token's slots here, only the first (and every slot of a local
// token); pass 1 copies the others from that first row, which by then is in xs
// (row_of, [R, K] = sorted position of every (row, slot) or -1, says which is which).
// dedup == 0: one pass, every row from its home.
__global__ void __launch_bounds__(256)
gather_rows_peer_kernel(bf16 *xs, const PeerRows src, int max_t,
                        const int *__restrict__ sorted_row,
                        const int *__restrict__ expert_offsets, int e_lo, int e_hi, int H, int R,
                        const int *__restrict__ row_of, int K, int rank, int dedup, int pass,
                        int *status) {
  // the rows of experts e_lo .. e_hi-1
  const int first = expert_offsets[e_lo], total = expert_offsets[e_hi];
  const int lane = threadIdx.x & 31;
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  const int n4 = H >> 3;
  for (int r = first + blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < total;
       r += nwarps) {
    const int g = sorted_row[r];
    if (g < 0 || g >= R) {
      if (pass == 0) set_status(status, kStatusBadIndex);
      continue;
    }
    const int home = g / max_t, tok = g - home * max_t;
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src.p[home] + static_cast<size_t>(tok) * H);
    if (dedup && home != rank) {
      // the first of this token's slots that landed on this rank
      int lead = -1;
      for (int k = 0; k < K && lead < 0; k++) lead = row_of[static_cast<size_t>(g) * K + k];
      const bool is_lead = lead == r || lead < 0;
      if (is_lead != (pass == 0)) continue;
      if (!is_lead) s4 = reinterpret_cast<const uint4 *>(xs + static_cast<size_t>(lead) * H);
    } else if (pass != 0) {
      continue;
    }
    uint4 *d4 = reinterpret_cast<uint4 *>(xs + static_cast<size_t>(r) * H);
    for (int p0 = lane; p0 < n4; p0 += 256) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; u++)
        if (p0 + u * 32 < n4) v[u] = s4[p0 + u * 32];  // (pass 1 reads xs itself: plain loads)
#pragma unroll
      for (int u = 0; u < 8; u++)
        if (p0 + u * 32 < n4) d4[p0 + u * 32] = v[u];
    }
  }
}

// 16 bytes that another GPU may have written while this kernel was already running (it
// spins on the flag that announces them): an ordinary relaxed load at system scope, not
// the read-only path, which is only defined for data that never changes under a kernel.
__device__ __forceinline__ uint4 ld_peer_v4(const uint4 *p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// x[t] = bf16(x[t] + sum over the token's K slots, in slot order, of the expert output row
// that the slot's owner holds for it).  Slot k of token t went to owner o = e % N, whose
// permutation put it at row_of[o][(rank * max_t + t) * K + k] of its sorted order; the
// owner's down GEMM left the weighted bf16 output there (ys).  Position and row are read
// from the owner's memory.  This is the sum the single-GPU combine makes, the same K rows
// in the same order, so sharding the experts adds no rounding of its own.
// One warp per token, two 16-byte columns per lane and trip.
// recv != nullptr: the owners' down GEMMs have stored the rows into this rank's receive buffer,
// slot (t, k) at row t * K + k: the same sum from local memory.
__global__ void __launch_bounds__(256)
combine_peer_kernel(bf16 *__restrict__ x, const PeerRows ys, const PeerInts rowof,
                    const bf16 *__restrict__ recv, const int *__restrict__ topk_i, int T, int K,
                    int N, int rank, int max_t, int H, int assign_cap, const int *flags, int round,
                    int *status, uint64_t limit_ns) {
  // every owner's outputs are complete (and every peer is done with this rank's activations);
  // a rank without tokens still takes this wait (one CTA): it is what allows it to
  // overwrite its published buffers in the next layer
  if (threadIdx.x < 32) ep_wait_flags(flags, N, round, status, limit_ns);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const bf16 *src[GPTOSS_MAX_TOPK];
  int nvalid = 0;
#pragma unroll
  for (int k = 0; k < GPTOSS_MAX_TOPK; k++) {
    src[k] = nullptr;
    if (k < K) {
      const int e = topk_i[t * K + k];
      if (e >= 0 && recv != nullptr) {
        src[k] = recv + (static_cast<size_t>(t) * K + k) * H;
        nvalid++;
      } else if (e >= 0) {
        const int o = e % N;
        int pos;
        asm volatile("ld.relaxed.sys.global.b32 %0, [%1];"
                     : "=r"(pos)
                     : "l"(rowof.p[o] + (static_cast<size_t>(rank) * max_t + t) * K + k)
                     : "memory");
        if (pos < 0 || pos >= assign_cap) {
          set_status(status, kStatusBadIndex);
        } else {
          src[k] = ys.p[o] + static_cast<size_t>(pos) * H;
          nvalid++;
        }
      }
    }
  }
  if (nvalid == 0) return;  // inactive row: x untouched
  uint4 *o4 = reinterpret_cast<uint4 *>(x + static_cast<size_t>(t) * H);
  const int n4 = H >> 3;
  for (int p0 = lane; p0 < n4; p0 += 64) {
    const int p1 = p0 + 32;
    const bool two = p1 < n4;
    uint4 xv[2], yv[2][GPTOSS_MAX_TOPK];
    xv[0] = o4[p0];
    xv[1] = two ? o4[p1] : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int k = 0; k < GPTOSS_MAX_TOPK; k++) {
      if (k < K && src[k]) {
        const uint4 *y4 = reinterpret_cast<const uint4 *>(src[k]);
        yv[0][k] = ld_peer_v4(y4 + p0);
        if (two) yv[1][k] = ld_peer_v4(y4 + p1);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; u++) {
      if (u == 1 && !two) break;
      float s[8];
#pragma unroll
      for (int i = 0; i < 8; i++) s[i] = 0.f;
#pragma unroll
      for (int k = 0; k < GPTOSS_MAX_TOPK; k++) {
        if (k < K && src[k]) {
          const uint4 v = yv[u][k];
          s[0] += bf16_lo(v.x); s[1] += bf16_hi(v.x); s[2] += bf16_lo(v.y); s[3] += bf16_hi(v.y);
          s[4] += bf16_lo(v.z); s[5] += bf16_hi(v.z); s[6] += bf16_lo(v.w); s[7] += bf16_hi(v.w);
        }
      }
      const uint4 v = xv[u];
      uint4 o;
      o.x = pack_bf16(bf16_lo(v.x) + s[0], bf16_hi(v.x) + s[1]);
      o.y = pack_bf16(bf16_lo(v.y) + s[2], bf16_hi(v.y) + s[3]);
      o.z = pack_bf16(bf16_lo(v.z) + s[4], bf16_hi(v.z) + s[5]);
      o.w = pack_bf16(bf16_lo(v.w) + s[6], bf16_hi(v.w) + s[7]);
      o4[u == 0 ? p0 : p1] = o;
    }
  }
}

// own_key[t, o] = o when token t has at least one selected expert on rank o.
__global__ void __launch_bounds__(256)
ep_owner_keys_kernel(const int *__restrict__ topk_i, int T, int K, int N,
                     int *__restrict__ own_key, float *__restrict__ own_w) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * N) return;
  const int t = i / N, o = i - t * N;
  bool has = false;
  for (int k = 0; k < K; k++) {
    const int e = topk_i[t * K + k];
    if (e >= 0 && e % N == o) has = true;
  }
  own_key[i] = has ? o : -1;
  own_w[i] = 0.f;
}

// One warp per send row p: copy the token's row and write its K slots as seen by
// the owner (local expert id e / N for the experts that live there, else -1).
__global__ void __launch_bounds__(256)
ep_pack_kernel(const bf16 *__restrict__ t, const int *__restrict__ topk_i,
               const float *__restrict__ topk_v, const int *__restrict__ s_offsets,
               const int *__restrict__ s_sorted_row, int N, int K, int H, int T,
               bf16 *__restrict__ send_rows, int *__restrict__ send_e,
               float *__restrict__ send_w, int *__restrict__ my_counts, int *status) {
  const int total = s_offsets[N];
  const int lane = threadIdx.x & 31;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  if (gw == 0 && lane < N) my_counts[lane] = s_offsets[lane + 1] - s_offsets[lane];
  const int n4 = H >> 3;
  for (int p = gw; p < total; p += nwarps) {
    const int tok = s_sorted_row[p];
    if (tok < 0 || tok >= T) {
      set_status(status, kStatusBadIndex);
      continue;
    }
    int owner = 0;
    while (owner + 1 < N && s_offsets[owner + 1] <= p) owner++;
    if (lane < K) {
      const int e = topk_i[tok * K + lane];
      const bool mine = e >= 0 && e % N == owner;
      send_e[static_cast<size_t>(p) * K + lane] = mine ? e / N : -1;
      send_w[static_cast<size_t>(p) * K + lane] = mine ? topk_v[tok * K + lane] : 0.f;
    }
    const uint4 *s4 = reinterpret_cast<const uint4 *>(t + static_cast<size_t>(tok) * H);
    uint4 *d4 = reinterpret_cast<uint4 *>(send_rows + static_cast<size_t>(p) * H);
    for (int q = lane; q < n4; q += 32) d4[q] = __ldg(s4 + q);
  }
}

// Checks the all-gathered row counts counts[src * N + dst] against the capacities every
// rank was created with; NULL when every rank can take part.
const char *ep_counts_problem(const int *counts, int N, int max_tokens, int send_cap,
                              int rows_cap) {
  for (int a = 0; a < N; a++) {
    long long sent = 0, received = 0;
    for (int b = 0; b < N; b++) {
      const int s = counts[a * N + b], r = counts[b * N + a];
      if (s < 0 || s > max_tokens) return "row counts exchanged between ranks are out of range";
      sent += s;
      received += r;
    }
    if (sent > send_cap || received > rows_cap)
      return "more rows routed than the engines were created for";
  }
  return nullptr;
}

static int ep_fail(gptoss_moe *h, int code, const std::string &msg) {
  h->err = msg;
  return code;
}

#define EP_CUDA(h, call)                                                                 \
  do {                                                                                   \
    cudaError_t e__ = (call);                                                            \
    if (e__ != cudaSuccess)                                                              \
      return ep_fail((h), GPTOSS_E_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__)); \
  } while (0)
#define EP_NCCL(h, call)                                                                 \
  do {                                                                                   \
    ncclResult_t r__ = (call);                                                           \
    if (r__ != ncclSuccess)                                                              \
      return ep_fail((h), GPTOSS_E_COMM, std::string(#call) + ": " + g_nccl.GetErrorString(r__)); \
  } while (0)

template <typename T>
static cudaError_t ep_alloc(T **p, size_t n) {
  return cudaMalloc(reinterpret_cast<void **>(p), (n ? n : 1) * sizeof(T));
}

struct EpStageScope {
  gptoss_moe *h;
  int id;
  cudaStream_t st;
  EpStageScope(gptoss_moe *h_, int id_, cudaStream_t st_) : h(h_), id(id_), st(st_) {
    if (!h->opt_time_stages) return;
    StageTimer &t = h->timers[id];
    if (t.used == t.beg.size()) {
      cudaEvent_t b, e;
      cudaEventCreate(&b);
      cudaEventCreate(&e);
      t.beg.push_back(b);
      t.end.push_back(e);
    }
    cudaEventRecord(t.beg[t.used], st);
  }
  ~EpStageScope() {
    if (!h->opt_time_stages) return;
    StageTimer &t = h->timers[id];
    cudaEventRecord(t.end[t.used], st);
    t.used++;
  }
};

// The layer over peer memory (see the head of this file), in three parts that one stream
// runs back to back.  A host that drives several ranks from ONE stream of one GPU (ranks as
// engines on the same device) can interleave them part by part - every rank's part 0, then
// every rank's part 1, then every rank's part 2 - and no kernel ever waits for a later
// launch; separate launches that wait for one another must never share a GPU otherwise.
static void peer_ctl_of(const EpState *ep, PeerCtl *ctl) {
  for (int p = 0; p < GPTOSS_MAX_TOPK; p++)
    ctl->p[p] = static_cast<int *>(p < ep->N ? ep->peer_ctl[p] : nullptr);
}

// part 0: publish - activations where the peers can read them, routing result into every
// rank's memory, then the flag "rank r of this round is in place"
static int ep_peer_publish(gptoss_moe *h, EpState *ep, const bf16 *t, int T, cudaStream_t st) {
  const int N = ep->N, K = h->K, H = h->H, max_t = ep->max_t;
  const int per = max_t * K;
  PeerCtl ctl;
  peer_ctl_of(ep, &ctl);
  const int round = ++ep->round;
  EpStageScope sc(h, 5, st);
  if (T > 0)
    EP_CUDA(h, cudaMemcpyAsync(ep->pub_t, t, static_cast<size_t>(T) * H * sizeof(bf16),
                               cudaMemcpyDeviceToDevice, st));
  ep_publish_meta_kernel<<<(per + 255) / 256, 256, 0, st>>>(h->topk_i, h->topk_v, T, max_t, K,
                                                            ctl, N, ep->rank);
  ep_signal_kernel<<<1, 32, 0, st>>>(ctl, N, 0, ep->rank, round);
  h->launches += 2;
  EP_CUDA(h, cudaGetLastError());
  return GPTOSS_OK;
}

// part 1: owner - wait for every rank's flag, sort all N * max_t rows by local expert, pull
// the rows out of the homes' memory (dispatch and gather in one kernel), both GEMMs, per-row
// sums, then the flag "my sums are complete"
static int ep_peer_owner(gptoss_moe *h, EpState *ep, int layer, const bf16 *t, cudaStream_t st) {
  const int N = ep->N, K = h->K, H = h->H, max_t = ep->max_t;
  const int per = max_t * K;
  const int round = ep->round;
  const uint64_t limit_ns = static_cast<uint64_t>(h->opt_wait_limit_ms) * 1000000ull;
  PeerCtl ctl;
  peer_ctl_of(ep, &ctl);
  {
    EpStageScope sc(h, 5, st);
    ep_owner_slots_kernel<<<(N * per + 255) / 256, 256, 0, st>>>(
        ep->all_meta, ep->ctl, round, N, ep->rank, max_t, K, ep->recv_e, ep->recv_w, h->status,
        limit_ns);
    h->launches++;
    EP_CUDA(h, cudaGetLastError());
  }
  const int R = N * max_t;
  h->stage_rows = nullptr;  // rows are pulled from the homes, not staged here
  h->stage_expert = ep->recv_e;
  h->stage_weight = ep->recv_w;
  h->stage_R = R;
  PeerRows src;
  for (int p = 0; p < GPTOSS_MAX_TOPK; p++)
    src.p[p] = static_cast<const bf16 *>(p < N ? ep->peer_t[p] : nullptr);
  if (t) src.p[ep->rank] = t;  // own rows straight from the caller's buffer
  // With the CTA-pair GEMM the experts can be taken in two halves: the rows of the second
  // half are pulled on a second stream while the first half is already being multiplied
  // (the gather kernel uses no shared memory and few registers, so its CTAs share the SMs
  // with the GEMM's).
  const bool halves = h->opt_ep_overlap && h->opt_gemm_impl == GPTOSS_GEMM_PAIR && h->El >= 2 && ep->s2;
  const int e_mid = halves ? h->El / 2 : h->El;
  {
    EpStageScope sc(h, 1, st);
    EP_CUDA(h, launch_permute_plan_only(h, st));
    if (halves) EP_CUDA(h, launch_mtile_split(h, e_mid, st));
    // (the copies of pass 1 read rows that pass 0 wrote, possibly for the other half of the
    // experts: no second pass when the gather is split)
    const int dedup = (h->opt_ep_dedup && !halves && K > 1) ? 1 : 0;
    gather_rows_peer_kernel<<<h->num_sms * 4, 256, 0, st>>>(h->xs, src, max_t, h->sorted_row,
                                                            h->expert_offsets, 0, e_mid, H, R,
                                                            h->row_of, K, ep->rank, dedup, 0,
                                                            h->status);
    h->launches++;
    EP_CUDA(h, cudaGetLastError());
    if (dedup) {
      gather_rows_peer_kernel<<<h->num_sms * 2, 256, 0, st>>>(h->xs, src, max_t, h->sorted_row,
                                                              h->expert_offsets, 0, e_mid, H, R,
                                                              h->row_of, K, ep->rank, dedup, 1,
                                                              h->status);
      h->launches++;
      EP_CUDA(h, cudaGetLastError());
    }
    if (halves) {
      // the second half starts when the first has the links to itself no longer
      EP_CUDA(h, cudaEventRecord(ep->ev_plan, st));
      EP_CUDA(h, cudaStreamWaitEvent(ep->s2, ep->ev_plan, 0));
      // few CTAs: the copy has to keep the links busy, not the SMs, which the GEMM needs
      gather_rows_peer_kernel<<<h->opt_ep_gather_ctas, 256, 0, ep->s2>>>(
          h->xs, src, max_t, h->sorted_row, h->expert_offsets, e_mid, h->El, H, R, h->row_of, K,
          ep->rank, 0, 0, h->status);
      EP_CUDA(h, cudaGetLastError());
      EP_CUDA(h, cudaEventRecord(ep->ev_second, ep->s2));
      h->launches++;
    }
  }
  {
    EpStageScope sc(h, 2, st);
    EP_CUDA(h, launch_gate_up(h, layer, st, halves ? 1 : 0));
    if (halves) {
      EP_CUDA(h, cudaStreamWaitEvent(st, ep->ev_second, 0));
      EP_CUDA(h, launch_gate_up(h, layer, st, 2));
    }
  }
  {
    EpStageScope sc(h, 3, st);
    const bool push = h->opt_ep_push && h->opt_gemm_impl == GPTOSS_GEMM_PAIR && ep->recv_out;
    if (push) {
      // every output row goes straight to the rank its token came from
      PeerBytes recv;
      for (int p = 0; p < GPTOSS_MAX_TOPK; p++)
        recv.p[p] = p < N ? reinterpret_cast<unsigned long long>(ep->peer_recv[p]) : 0ull;
      ep_row_dst_kernel<<<(N * per + 255) / 256, 256, 0, st>>>(h->row_of, recv, N, per, H,
                                                               h->assign_cap, h->row_dst);
      h->launches++;
      EP_CUDA(h, cudaGetLastError());
    }
    h->push_rows = push;
    const cudaError_t e_down = launch_down(h, layer, st);
    h->push_rows = false;
    EP_CUDA(h, e_down);
  }
  {
    // the homes read the expert outputs where the down GEMM left them (or find them in their
    // own receive buffers): "my outputs are complete" goes out right behind it
    EpStageScope sc(h, 6, st);
    ep_signal_kernel<<<1, 32, 0, st>>>(ctl, N, 1, ep->rank, round);
    h->launches++;
    EP_CUDA(h, cudaGetLastError());
  }
  return GPTOSS_OK;
}

// part 2: home - wait for every owner's flag, pull the sums of this rank's tokens and add
// them and the residual (return and combine in one kernel).  Without tokens the kernel is
// still launched, with one CTA, for its wait: the second flags are also the proof that
// every peer has finished reading this rank's published buffers.
static int ep_peer_combine(gptoss_moe *h, EpState *ep, void *x_io, int T, cudaStream_t st) {
  const int N = ep->N, K = h->K, H = h->H, max_t = ep->max_t;
  const uint64_t limit_ns = static_cast<uint64_t>(h->opt_wait_limit_ms) * 1000000ull;
  PeerRows outs;
  PeerInts rowof;
  for (int p = 0; p < GPTOSS_MAX_TOPK; p++) {
    outs.p[p] = static_cast<const bf16 *>(p < N ? ep->peer_out[p] : nullptr);
    rowof.p[p] = static_cast<const int *>(p < N ? ep->peer_rowof[p] : nullptr);
  }
  EpStageScope sc(h, 4, st);
  const int warps = 8;
  const int grid = T > 0 ? (T + warps - 1) / warps : 1;
  const bool pushed = h->opt_ep_push && h->opt_gemm_impl == GPTOSS_GEMM_PAIR && ep->recv_out;
  combine_peer_kernel<<<grid, warps * 32, 0, st>>>(static_cast<bf16 *>(x_io), outs, rowof,
                                                   pushed ? ep->recv_out : nullptr,
                                                   h->topk_i, T, K, N, ep->rank, max_t, H,
                                                   h->assign_cap, ep->ctl + N, ep->round, h->status,
                                                   limit_ns);
  h->launches++;
  EP_CUDA(h, cudaGetLastError());
  return GPTOSS_OK;
}

static int ep_forward_peer(gptoss_moe *h, EpState *ep, int layer, const bf16 *t, void *x_io, int T,
                           cudaStream_t st) {
  int rc = ep_peer_publish(h, ep, t, T, st);
  if (rc) return rc;
  if ((rc = ep_peer_owner(h, ep, layer, t, st))) return rc;
  return ep_peer_combine(h, ep, x_io, T, st);
}

int ep_forward_part(gptoss_moe *h, int layer, int part, const void *t, void *x_io, int T,
                    void *stream) {
  EpState *ep = static_cast<EpState *>(h->ep);
  if (!ep || !ep->peer_ok || ep->transport != 1)
    return ep_fail(h, GPTOSS_E_STATE, "the layer runs in parts only over the peer-memory transport");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (part) {
    case 0: return ep_peer_publish(h, ep, static_cast<const bf16 *>(t), T, st);
    case 1: return ep_peer_owner(h, ep, layer, static_cast<const bf16 *>(t), st);
    case 2: return ep_peer_combine(h, ep, x_io, T, st);
    default: return ep_fail(h, GPTOSS_E_INVALID, "part must be 0, 1 or 2");
  }
}

int ep_set_transport(gptoss_moe *h, int transport) {
  EpState *ep = static_cast<EpState *>(h->ep);
  if (!ep) return ep_fail(h, GPTOSS_E_STATE, "expert parallelism is not set up");
  if (transport != 0 && transport != 1)
    return ep_fail(h, GPTOSS_E_INVALID, "ep_transport: 0 = NCCL send/recv, 1 = peer memory");
  if (transport == 1 && !ep->peer_ok)
    return ep_fail(h, GPTOSS_E_STATE, "peer-memory transport unavailable: " + ep->peer_why);
  if (transport == 0 && !ep->comm)
    return ep_fail(h, GPTOSS_E_STATE, "NCCL transport unavailable: the ranks were wired inside "
                                      "one process without a communicator");
  ep->transport = transport;
  return GPTOSS_OK;
}

int ep_get_transport(const gptoss_moe *h) {
  const EpState *ep = static_cast<const EpState *>(h->ep);
  return ep ? ep->transport : -1;
}

int ep_forward(gptoss_moe *h, int layer, const void *t_in, void *x_io, int T, void *stream) {
  EpState *ep = static_cast<EpState *>(h->ep);
  if (!ep || (!ep->comm && !ep->peer_ok))
    return ep_fail(h, GPTOSS_E_STATE,
                   "expert parallelism is not set up: call gptoss_moe_ep_init first");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ep->transport == 1)
    return ep_forward_peer(h, ep, layer, static_cast<const bf16 *>(t_in), x_io, T, st);
  if (!ep->comm) return ep_fail(h, GPTOSS_E_STATE, "no NCCL communicator on this engine");
  const int N = ep->N, K = h->K, H = h->H;
  const bf16 *t = static_cast<const bf16 *>(t_in);
  std::vector<int> soff(N + 1, 0), roff(N + 1, 0);
  {
    EpStageScope sc(h, 5, st);
    // 1. per-owner send lists
    if (T > 0) {
      ep_owner_keys_kernel<<<(T * N + 255) / 256, 256, 0, st>>>(h->topk_i, T, K, N, ep->own_key,
                                                                ep->own_w);
      h->launches++;
      EP_CUDA(h, cudaGetLastError());
    }
    PermPlan p;
    p.slot_expert = ep->own_key;
    p.slot_weight = ep->own_w;
    p.R = T; p.K = N; p.El = N;
    p.block_counts = ep->s_block_counts;
    p.blocks_cap = ep->s_blocks_cap;
    p.expert_offsets = ep->s_offsets;
    p.sorted_row = ep->s_sorted_row;
    p.sorted_weight = ep->s_sorted_w;
    p.row_of = ep->s_row_of;
    p.mtile_expert = ep->s_mtile;
    p.mtile_row0 = ep->s_mtile + ep->s_mtiles_cap;
    p.mtile_rows = ep->s_mtile + 2 * ep->s_mtiles_cap;
    p.num_mtiles = ep->s_mtile + 3 * ep->s_mtiles_cap;
    p.mtiles_cap = ep->s_mtiles_cap;
    p.assign_cap = ep->send_cap;
    EP_CUDA(h, launch_perm_plan(p, h->status, st, &h->launches));
    ep_pack_kernel<<<h->num_sms * 4, 256, 0, st>>>(t, h->topk_i, h->topk_v, ep->s_offsets,
                                                   ep->s_sorted_row, N, K, H, T, ep->send_rows,
                                                   ep->send_e, ep->send_w,
                                                   ep->counts_dev + ep->rank * N, h->status);
    h->launches++;
    EP_CUDA(h, cudaGetLastError());
    // 2. counts to every rank, then to the host
    EP_NCCL(h, g_nccl.AllGather(ep->counts_dev + ep->rank * N, ep->counts_dev, N, ncclInt32,
                                ep->comm, st));
    EP_CUDA(h, cudaMemcpyAsync(ep->counts_host, ep->counts_dev, sizeof(int) * N * N,
                               cudaMemcpyDeviceToHost, st));
    EP_CUDA(h, cudaStreamSynchronize(st));
    // go / no-go from the whole N x N matrix, which every rank holds: all ranks decide
    // alike (max_tokens is the same everywhere, gptoss_moe_ep_init checked it), so none
    // leaves the others inside a grouped send / recv that can never be matched
    {
      const char *why = ep_counts_problem(ep->counts_host, N, h->max_tokens, ep->send_cap,
                                          h->rows_cap);
      if (why) return ep_fail(h, GPTOSS_E_CAPACITY, why);
    }
    for (int p2 = 0; p2 < N; p2++) {
      soff[p2 + 1] = soff[p2] + ep->counts_host[ep->rank * N + p2];
      roff[p2 + 1] = roff[p2] + ep->counts_host[p2 * N + ep->rank];
    }
    // 3. dispatch
    EP_NCCL(h, g_nccl.GroupStart());
    for (int p2 = 0; p2 < N; p2++) {
      const size_t s = soff[p2 + 1] - soff[p2], r = roff[p2 + 1] - roff[p2];
      if (s) {
        EP_NCCL(h, g_nccl.Send(ep->send_rows + (size_t)soff[p2] * H, s * H, ncclBfloat16, p2,
                               ep->comm, st));
        EP_NCCL(h, g_nccl.Send(ep->send_e + (size_t)soff[p2] * K, s * K, ncclInt32, p2, ep->comm,
                               st));
        EP_NCCL(h, g_nccl.Send(ep->send_w + (size_t)soff[p2] * K, s * K, ncclFloat32, p2,
                               ep->comm, st));
      }
      if (r) {
        EP_NCCL(h, g_nccl.Recv(ep->recv_rows + (size_t)roff[p2] * H, r * H, ncclBfloat16, p2,
                               ep->comm, st));
        EP_NCCL(h, g_nccl.Recv(ep->recv_e + (size_t)roff[p2] * K, r * K, ncclInt32, p2, ep->comm,
                               st));
        EP_NCCL(h, g_nccl.Recv(ep->recv_w + (size_t)roff[p2] * K, r * K, ncclFloat32, p2,
                               ep->comm, st));
      }
    }
    EP_NCCL(h, g_nccl.GroupEnd());
  }
  // 4. owner: this rank's experts on everything received
  const int R = roff[N];
  h->stage_rows = ep->recv_rows;
  h->stage_expert = ep->recv_e;
  h->stage_weight = ep->recv_w;
  h->stage_R = R;
  {
    EpStageScope sc(h, 1, st);
    EP_CUDA(h, launch_permute(h, st));
  }
  {
    EpStageScope sc(h, 2, st);
    EP_CUDA(h, launch_gate_up(h, layer, st));
  }
  {
    EpStageScope sc(h, 3, st);
    EP_CUDA(h, launch_down(h, layer, st));
  }
  {
    EpStageScope sc(h, 6, st);
    EP_CUDA(h, launch_reduce_rows(h, ep->out_rows, R, st));
    // 5. return the per-row sums to the homes
    EP_NCCL(h, g_nccl.GroupStart());
    for (int p2 = 0; p2 < N; p2++) {
      const size_t s = soff[p2 + 1] - soff[p2], r = roff[p2 + 1] - roff[p2];
      if (r)
        EP_NCCL(h, g_nccl.Send(ep->out_rows + (size_t)roff[p2] * H, r * H, ncclBfloat16, p2,
                               ep->comm, st));
      if (s)
        EP_NCCL(h, g_nccl.Recv(ep->ret_rows + (size_t)soff[p2] * H, s * H, ncclBfloat16, p2,
                               ep->comm, st));
    }
    EP_NCCL(h, g_nccl.GroupEnd());
  }
  {
    // 6. home: one returned row per (token, owner)
    EpStageScope sc(h, 4, st);
    EP_CUDA(h, launch_combine_rows(true, static_cast<bf16 *>(x_io), ep->ret_rows, ep->s_row_of, T,
                                   N, H, ep->send_cap, h->status, st, &h->launches));
  }
  return GPTOSS_OK;
}

struct PeerBlob {  // what a rank tells the others at start-up
  cudaIpcMemHandle_t t, out, rowof, ctl, recv;
  int ok, max_t, hidden, pid, top_k, experts;
};

static int ep_map_peers(gptoss_moe *h, EpState *ep) {
  const int N = ep->N;
  PeerBlob mine = {};
  mine.max_t = ep->max_t;
  mine.hidden = h->H;
  mine.top_k = h->K;
  mine.experts = h->E;
  mine.pid = static_cast<int>(getpid());
  mine.ok = cudaIpcGetMemHandle(&mine.t, ep->pub_t) == cudaSuccess &&
            cudaIpcGetMemHandle(&mine.out, h->ys) == cudaSuccess &&
            cudaIpcGetMemHandle(&mine.rowof, h->row_of) == cudaSuccess &&
            cudaIpcGetMemHandle(&mine.ctl, ep->ctl) == cudaSuccess &&
            cudaIpcGetMemHandle(&mine.recv, ep->recv_out) == cudaSuccess;
  if (!mine.ok) {
    ep->peer_why = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(cudaGetLastError());
  }
  static_assert(sizeof(PeerBlob) % 4 == 0, "exchanged as 32-bit words");
  PeerBlob *blobs_dev = nullptr;
  std::vector<PeerBlob> blobs(N);
  EP_CUDA(h, ep_alloc(&blobs_dev, (size_t)N));
  EP_CUDA(h, cudaMemcpy(blobs_dev + ep->rank, &mine, sizeof(mine), cudaMemcpyHostToDevice));
  EP_NCCL(h, g_nccl.AllGather(blobs_dev + ep->rank, blobs_dev, sizeof(PeerBlob) / 4, ncclInt32,
                              ep->comm, nullptr));
  EP_CUDA(h, cudaStreamSynchronize(nullptr));
  EP_CUDA(h, cudaMemcpy(blobs.data(), blobs_dev, sizeof(PeerBlob) * N, cudaMemcpyDeviceToHost));
  // engines that do not agree on their sizes cannot work together over either transport:
  // every rank sees the same blobs, so every rank fails here, before any other exchange
  for (int p = 0; p < N; p++) {
    if (blobs[p].max_t != ep->max_t || blobs[p].hidden != h->H || blobs[p].top_k != h->K ||
        blobs[p].experts != h->E) {
      cudaFree(blobs_dev);
      return ep_fail(h, GPTOSS_E_INVALID,
                     "ranks were created with different max_tokens, hidden size, expert count "
                     "or top-k");
    }
  }
  bool ok = true;
  for (int p = 0; p < N && ok; p++) {
    if (!blobs[p].ok) {
      ok = false;
      if (ep->peer_why.empty()) ep->peer_why = "a peer rank could not export its buffers";
    } else if (p != ep->rank && blobs[p].pid == mine.pid) {
      ok = false;
      ep->peer_why = "ranks share a process (IPC mappings need one process per rank)";
    }
  }
  for (int p = 0; p < N && ok; p++) {
    if (p == ep->rank) {
      ep->peer_t[p] = ep->pub_t;
      ep->peer_out[p] = h->ys;
      ep->peer_rowof[p] = h->row_of;
      ep->peer_ctl[p] = ep->ctl;
      ep->peer_recv[p] = ep->recv_out;
      continue;
    }
    cudaError_t e = cudaIpcOpenMemHandle(&ep->peer_t[p], blobs[p].t, cudaIpcMemLazyEnablePeerAccess);
    if (e == cudaSuccess)
      e = cudaIpcOpenMemHandle(&ep->peer_out[p], blobs[p].out, cudaIpcMemLazyEnablePeerAccess);
    if (e == cudaSuccess)
      e = cudaIpcOpenMemHandle(&ep->peer_rowof[p], blobs[p].rowof, cudaIpcMemLazyEnablePeerAccess);
    if (e == cudaSuccess)
      e = cudaIpcOpenMemHandle(&ep->peer_ctl[p], blobs[p].ctl, cudaIpcMemLazyEnablePeerAccess);
    if (e == cudaSuccess)
      e = cudaIpcOpenMemHandle(&ep->peer_recv[p], blobs[p].recv, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      ok = false;
      ep->peer_why = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e);
      cudaGetLastError();
    }
  }
  // second round: the transport is usable only if every rank mapped every peer
  int mapped = ok ? 1 : 0;
  int *flags_dev = reinterpret_cast<int *>(blobs_dev);
  std::vector<int> flags(N, 0);
  EP_CUDA(h, cudaMemcpy(flags_dev + ep->rank, &mapped, sizeof(int), cudaMemcpyHostToDevice));
  EP_NCCL(h, g_nccl.AllGather(flags_dev + ep->rank, flags_dev, 1, ncclInt32, ep->comm, nullptr));
  EP_CUDA(h, cudaStreamSynchronize(nullptr));
  EP_CUDA(h, cudaMemcpy(flags.data(), flags_dev, sizeof(int) * N, cudaMemcpyDeviceToHost));
  cudaFree(blobs_dev);
  for (int p = 0; p < N; p++)
    if (!flags[p]) {
      ok = false;
      if (ep->peer_why.empty()) ep->peer_why = "a peer rank could not map this rank's buffers";
    }
  ep->peer_ok = ok;
  ep->transport = ok ? 1 : 0;
  return GPTOSS_OK;
}

void ep_destroy(gptoss_moe *h) {
  EpState *ep = static_cast<EpState *>(h->ep);
  if (!ep) return;
  for (int p = 0; p < ep->N && !ep->local; p++) {
    if (p == ep->rank) continue;
    if (ep->peer_t[p]) cudaIpcCloseMemHandle(ep->peer_t[p]);
    if (ep->peer_out[p]) cudaIpcCloseMemHandle(ep->peer_out[p]);
    if (ep->peer_rowof[p]) cudaIpcCloseMemHandle(ep->peer_rowof[p]);
    if (ep->peer_ctl[p]) cudaIpcCloseMemHandle(ep->peer_ctl[p]);
    if (ep->peer_recv[p]) cudaIpcCloseMemHandle(ep->peer_recv[p]);
  }
  cudaFree(ep->pub_t); cudaFree(ep->ctl); cudaFree(ep->recv_out);
  if (ep->s2) cudaStreamDestroy(ep->s2);
  if (ep->ev_plan) cudaEventDestroy(ep->ev_plan);
  if (ep->ev_second) cudaEventDestroy(ep->ev_second);
  if (ep->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(ep->comm);
  cudaFree(ep->own_key); cudaFree(ep->own_w); cudaFree(ep->s_block_counts);
  cudaFree(ep->s_offsets); cudaFree(ep->s_sorted_row); cudaFree(ep->s_sorted_w);
  cudaFree(ep->s_row_of); cudaFree(ep->s_mtile); cudaFree(ep->send_rows); cudaFree(ep->send_e);
  cudaFree(ep->send_w); cudaFree(ep->ret_rows); cudaFree(ep->recv_rows); cudaFree(ep->recv_e);
  cudaFree(ep->recv_w); cudaFree(ep->out_rows); cudaFree(ep->counts_dev);
  if (ep->counts_host) cudaFreeHost(ep->counts_host);
  delete ep;
  h->ep = nullptr;
}

}  // namespace gptoss

using namespace gptoss;

extern "C" int gptoss_moe_ep_unique_id(void *id128) {
  if (!id128) return GPTOSS_E_INVALID;
  std::string err;
  if (!load_nccl(&err)) return set_global_error(GPTOSS_E_COMM, err.c_str());
  static_assert(sizeof(ncclUniqueId) == 128, "id buffer size");
  ncclUniqueId id;
  ncclResult_t r = g_nccl.GetUniqueId(&id);
  if (r != ncclSuccess) return set_global_error(GPTOSS_E_COMM, g_nccl.GetErrorString(r));
  memcpy(id128, &id, sizeof(id));
  return GPTOSS_OK;
}

// Buffers of the peer-memory transport (also the owner-side staging both transports use).
static int ep_alloc_peer_side(gptoss_moe *h, EpState *ep) {
  const int N = ep->N, K = h->K, H = h->H;
  const size_t T = h->max_tokens;
  ep->max_t = static_cast<int>(T);
  EP_CUDA(h, ep_alloc(&ep->recv_e, (size_t)h->rows_cap * K));
  EP_CUDA(h, ep_alloc(&ep->recv_w, (size_t)h->rows_cap * K));
  EP_CUDA(h, ep_alloc(&ep->pub_t, T * H));
  EP_CUDA(h, ep_alloc(&ep->recv_out, T * K * H));
  if (!h->row_dst) EP_CUDA(h, ep_alloc(&h->row_dst, (size_t)h->assign_cap));
  EP_CUDA(h, ep_alloc(&ep->ctl, (size_t)kCtlHeader + (size_t)N * 2 * T * K));
  EP_CUDA(h, cudaMemset(ep->ctl, 0, sizeof(int) * kCtlHeader));
  ep->all_meta = ep->ctl + kCtlHeader;
  // expert ids of a rank that has not published yet read as -1 (no row), not as garbage
  EP_CUDA(h, cudaMemset(ep->all_meta, 0xFF, sizeof(int) * (size_t)N * 2 * T * K));
  EP_CUDA(h, cudaStreamCreateWithFlags(&ep->s2, cudaStreamNonBlocking));
  EP_CUDA(h, cudaEventCreateWithFlags(&ep->ev_plan, cudaEventDisableTiming));
  EP_CUDA(h, cudaEventCreateWithFlags(&ep->ev_second, cudaEventDisableTiming));
  return GPTOSS_OK;
}

extern "C" int gptoss_moe_ep_init(gptoss_moe_t *h, const void *id128) {
  if (!h || !id128) return GPTOSS_E_INVALID;
  if (h->ep_size <= 1) return ep_fail(h, GPTOSS_E_STATE, "engine was created with ep_size <= 1");
  if (h->ep) return ep_fail(h, GPTOSS_E_STATE, "expert parallelism already set up");
  if (h->ep_size > GPTOSS_MAX_TOPK)
    return ep_fail(h, GPTOSS_E_INVALID, "at most 8 ranks (one combine slot per owner)");
  std::string err;
  if (!load_nccl(&err)) return ep_fail(h, GPTOSS_E_COMM, err);
  EP_CUDA(h, cudaSetDevice(h->cfg.device));
  EpState *ep = new EpState();
  h->ep = ep;
  ep->N = h->ep_size;
  ep->rank = h->ep_rank;
  const int N = ep->N, K = h->K, H = h->H;
  const size_t T = h->max_tokens;
  ep->send_cap = static_cast<int>(T) * (N < K ? N : K);
  ep->s_blocks_cap = (static_cast<int>(T) + kPermTokens - 1) / kPermTokens;
  ep->s_mtiles_cap = ep->send_cap / kTileM + N + 1;
  EP_CUDA(h, ep_alloc(&ep->own_key, T * N));
  EP_CUDA(h, ep_alloc(&ep->own_w, T * N));
  EP_CUDA(h, ep_alloc(&ep->s_block_counts, (size_t)ep->s_blocks_cap * N));
  EP_CUDA(h, ep_alloc(&ep->s_offsets, (size_t)N + 1));
  EP_CUDA(h, ep_alloc(&ep->s_sorted_row, (size_t)ep->send_cap));
  EP_CUDA(h, ep_alloc(&ep->s_sorted_w, (size_t)ep->send_cap));
  EP_CUDA(h, ep_alloc(&ep->s_row_of, T * N));
  EP_CUDA(h, ep_alloc(&ep->s_mtile, (size_t)3 * ep->s_mtiles_cap + 1));
  EP_CUDA(h, ep_alloc(&ep->send_rows, (size_t)ep->send_cap * H));
  EP_CUDA(h, ep_alloc(&ep->send_e, (size_t)ep->send_cap * K));
  EP_CUDA(h, ep_alloc(&ep->send_w, (size_t)ep->send_cap * K));
  EP_CUDA(h, ep_alloc(&ep->ret_rows, (size_t)ep->send_cap * H));
  EP_CUDA(h, ep_alloc(&ep->recv_rows, (size_t)h->rows_cap * H));
  EP_CUDA(h, ep_alloc(&ep->out_rows, (size_t)h->rows_cap * H));
  EP_CUDA(h, ep_alloc(&ep->counts_dev, (size_t)N * N));
  EP_CUDA(h, cudaMemset(ep->counts_dev, 0, sizeof(int) * N * N));
  EP_CUDA(h, cudaMemset(ep->s_offsets, 0, sizeof(int) * (N + 1)));
  EP_CUDA(h, cudaMallocHost(reinterpret_cast<void **>(&ep->counts_host), sizeof(int) * N * N));
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  EP_NCCL(h, g_nccl.CommInitRank(&ep->comm, N, id, ep->rank));
  // peer-memory transport: buffers the peers map, handles exchanged over the new
  // communicator.  Every rank takes part in the exchange whatever happens locally, so a
  // rank that cannot export or map memory does not leave the others waiting; the
  // transport is offered only when every rank mapped every peer.
  int rc = ep_alloc_peer_side(h, ep);
  if (rc) return rc;
  return ep_map_peers(h, ep);
}

// All ranks live in this process (one host thread per GPU, the reference's own host shape,
// getp_run.cpp:1038-1063): no communicator and no IPC handles are needed, the engines learn
// each other's buffers as plain pointers once peer access between their devices is on.
extern "C" int gptoss_moe_ep_init_local(gptoss_moe_t *const *engines, int n_engines) {
  if (!engines || n_engines < 2 || n_engines > GPTOSS_MAX_TOPK)
    return set_global_error(GPTOSS_E_INVALID, "gptoss_moe_ep_init_local: 2 to 8 engines");
  const int N = n_engines;
  for (int r = 0; r < N; r++) {
    gptoss_moe *h = engines[r];
    if (!h) return set_global_error(GPTOSS_E_INVALID, "gptoss_moe_ep_init_local: null engine");
    if (h->ep) return ep_fail(h, GPTOSS_E_STATE, "expert parallelism already set up");
    if (h->ep_size != N || h->ep_rank != r)
      return ep_fail(h, GPTOSS_E_INVALID, "engines[r] must have been created with ep_rank r and "
                                          "ep_size n_engines");
    const gptoss_moe *h0 = engines[0];
    if (h->max_tokens != h0->max_tokens || h->H != h0->H || h->K != h0->K || h->E != h0->E)
      return ep_fail(h, GPTOSS_E_INVALID,
                     "ranks were created with different max_tokens, hidden size, expert count "
                     "or top-k");
  }
  // peer access between every pair of distinct devices
  for (int a = 0; a < N; a++) {
    for (int b = 0; b < N; b++) {
      const int da = engines[a]->cfg.device, db = engines[b]->cfg.device;
      if (da == db) continue;
      int can = 0;
      cudaError_t e = cudaDeviceCanAccessPeer(&can, da, db);
      if (e != cudaSuccess || !can)
        return ep_fail(engines[a], GPTOSS_E_CUDA, "no peer access between the engines' devices");
      if ((e = cudaSetDevice(da)) != cudaSuccess)
        return ep_fail(engines[a], GPTOSS_E_CUDA, cudaGetErrorString(e));
      e = cudaDeviceEnablePeerAccess(db, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
      } else if (e != cudaSuccess) {
        return ep_fail(engines[a], GPTOSS_E_CUDA,
                       std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e));
      }
    }
  }
  int rc = GPTOSS_OK;
  for (int r = 0; r < N && rc == GPTOSS_OK; r++) {
    gptoss_moe *h = engines[r];
    if (cudaSetDevice(h->cfg.device) != cudaSuccess) {
      rc = ep_fail(h, GPTOSS_E_CUDA, "cudaSetDevice");
      break;
    }
    EpState *ep = new EpState();
    h->ep = ep;
    ep->N = N;
    ep->rank = r;
    ep->local = true;
    rc = ep_alloc_peer_side(h, ep);
    if (rc == GPTOSS_OK && cudaDeviceSynchronize() != cudaSuccess)
      rc = ep_fail(h, GPTOSS_E_CUDA, "cudaDeviceSynchronize");
  }
  if (rc != GPTOSS_OK) {
    for (int r = 0; r < N; r++)
      if (engines[r]->ep) {
        cudaSetDevice(engines[r]->cfg.device);
        ep_destroy(engines[r]);
      }
    return rc;
  }
  for (int r = 0; r < N; r++) {
    EpState *ep = static_cast<EpState *>(engines[r]->ep);
    for (int p = 0; p < N; p++) {
      EpState *peer = static_cast<EpState *>(engines[p]->ep);
      ep->peer_t[p] = peer->pub_t;
      ep->peer_out[p] = engines[p]->ys;
      ep->peer_rowof[p] = engines[p]->row_of;
      ep->peer_ctl[p] = peer->ctl;
      ep->peer_recv[p] = peer->recv_out;
    }
    ep->peer_ok = true;
    ep->transport = 1;
  }
  return GPTOSS_OK;
}

extern "C" int gptoss_moe_forward_part(gptoss_moe_t *h, int layer, int part, const void *t, void *x,
                                       const int *pos, int n_tokens, void *stream) {
  if (!h) return GPTOSS_E_INVALID;
  if (layer < 0 || layer >= h->L || !h->layers[layer].loaded)
    return ep_fail(h, GPTOSS_E_STATE, "layer out of range or not loaded");
  if (n_tokens < 0 || n_tokens > h->max_tokens)
    return ep_fail(h, GPTOSS_E_CAPACITY, "n_tokens out of range");
  if ((part == 0 && !t && n_tokens > 0) || (part == 2 && !x && n_tokens > 0))
    return ep_fail(h, GPTOSS_E_INVALID, "null activation pointer");
  EP_CUDA(h, cudaSetDevice(h->cfg.device));
  if (part == 0) {
    int rc = gptoss_moe_route(h, layer, t, pos, n_tokens, stream);
    if (rc) return rc;
  }
  return ep_forward_part(h, layer, part, t, x, n_tokens, stream);
}

// Not part of the public header: lets host-side tests put the capacity check of the NCCL
// transport in front of count matrices of their own (pure host code, no GPU needed).
extern "C" const char *gptoss_internal_ep_counts_problem(const int *counts, int n_ranks,
                                                         int max_tokens, int top_k) {
  const int send_cap = max_tokens * (n_ranks < top_k ? n_ranks : top_k);
  return ep_counts_problem(counts, n_ranks, max_tokens, send_cap, max_tokens * n_ranks);
}

extern "C" int gptoss_moe_ep_transport(const gptoss_moe_t *h) {
  if (!h) return -1;
  return ep_get_transport(h);
}
