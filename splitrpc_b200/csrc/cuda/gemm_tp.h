// Launch API of the tensor-parallel fused kernels (all-gather -> GEMM, GEMM ->
// reduce-scatter, reduce + LayerNorm) over NVLink peer memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_tcgen05.h"

#define TP_MAX_RANKS 8

struct TpParams {
  int tp = 1, rank = 0;
  uint32_t epoch = 0;            // flags are monotonically increasing step numbers
  const uint32_t* epoch_base = nullptr;  // optional device word added to `epoch` at run time (lets a captured
                                         // graph use fresh step numbers on every replay)
  // ---- all-gather side (mblock_ready == nullptr: A is entirely local)
  uint32_t* mblock_ready = nullptr;  // local flags, one per 128-row block of A
  int n_copy = 0;                    // copier blocks appended to the grid
  const uint8_t* src[TP_MAX_RANKS] = {};  // src[r]: rank r's own shard (rows r*M/tp ...) in r's memory
  uint8_t* gathered = nullptr;       // local A buffer [M, K]; this rank's shard is already in place
  const uint32_t* src_ready = nullptr;  // local words [tp]: peers publish their shard's epoch here
  // ---- reduce-scatter side (rs == 0: plain local output)
  int rs = 0;
  uint8_t* dst[TP_MAX_RANKS] = {};       // dst[o]: slot for this rank's partial rows on owner o ([M/tp, ldo])
  uint32_t* dst_flag[TP_MAX_RANKS] = {};  // dst_flag[o]: word on owner o that receives the epoch when all tiles are there
  uint32_t* owner_count = nullptr;       // local zeroed counters [tp]
  // ---- filled in by the launcher
  int mblocks_per_rank = 0, m_rot = 0, tiles_per_owner = 0;
  size_t mblock_bytes = 0;
};

struct TpSignal {
  int tp;
  uint32_t epoch;
  const uint32_t* epoch_base;
  uint32_t* peer_flag[TP_MAX_RANKS];  // peer_flag[p]: this rank's word in peer p's signal area
};

struct TpReduce {
  int tp, hidden;
  uint32_t epoch;
  const uint32_t* epoch_base;
  const uint32_t* flags;                       // local words [tp] written by the source ranks
  const __nv_bfloat16* slots[TP_MAX_RANKS];    // local partial buffers, one per source rank, [rows, hidden]
  const float* bias;
  const __nv_bfloat16* residual;               // [rows, hidden] or null
  const float *gamma, *beta;
  __nv_bfloat16* out;
  float eps;
  // Optional: when the last block has written its rows, publish `sig_epoch` (+ *epoch_base) in every peer's flag word,
  // so that no separate signalling launch is needed.  `done_count` is a zeroed device word owned by the caller.
  int sig_tp;
  uint32_t sig_epoch;
  uint32_t* sig_peer_flag[TP_MAX_RANKS];
  uint32_t* done_count;
};

// D = act(A . B^T + bias); A is [M, K] with M/128 divisible by tp.  With tp.mblock_ready set, remote row blocks of A
// are pulled into tp.gathered by copier blocks of the same launch (N == 0 gives a pure all-gather).  With tp.rs set,
// finished tiles are stored into the owners' slots instead of ep.out (ep.ldo = row stride of a slot).
cudaError_t srpc_gemm_tp(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const GemmEpilogue& ep,
                         const TpParams& tp, uint32_t* status, cudaStream_t stream);
// The same operation on 256-row tiles computed by CTA pairs (tcgen05 cta_group::2); srpc_gemm_tp forwards the shapes
// that srpc_gemm_tp_2sm_eligible accepts (rows per rank a multiple of 256, N >= 128) unless SPLITRPC_TP_2SM=0.
bool srpc_gemm_tp_2sm_eligible(int M, int N, int K, const GemmEpilogue& ep, const TpParams& tp);
cudaError_t srpc_gemm_tp_2sm(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const GemmEpilogue& ep,
                             const TpParams& tp, uint32_t* status, cudaStream_t stream);
cudaError_t srpc_gemm_tp_2sm_set_wait_ns(uint64_t ns);
cudaError_t srpc_tp_signal(const TpSignal& sig, cudaStream_t stream);
// Stream-ordered bounded wait until flags[0..n) >= epoch (+ *epoch_base); a timeout sets *status.
cudaError_t srpc_tp_wait(const uint32_t* flags, int n, uint32_t epoch, const uint32_t* epoch_base, uint32_t* status,
                         cudaStream_t stream);
// srpc_tp_wait(flags, n, 0, epoch_base) followed by srpc_tp_bump(epoch_base, delta), as one launch.
cudaError_t srpc_tp_begin(const uint32_t* flags, int n, uint32_t* epoch_base, uint32_t delta, uint32_t* status,
                          cudaStream_t stream);
// *word += delta, stream ordered (advances the step-number base between forward passes).
cudaError_t srpc_tp_bump(uint32_t* word, uint32_t delta, cudaStream_t stream);
cudaError_t srpc_layernorm_reduce(const TpReduce& rd, int rows, uint32_t* status, cudaStream_t stream);

// Request fan-out of a tensor-parallel replica: the rank that owns the request ring stores the batch's requests into
// every rank's input buffer (its own included) over peer memory, then a two-word control record {command, batch} and,
// with a system-scope release store, the next sequence number into every rank's doorbell word.  The other ranks'
// streams are parked on that word (cuStreamWaitValue32, >=), so no host thread and no collective library sits between
// the arrival of a batch and the start of the model on any rank.
struct TpFanout {
  int tp;
  const void* stub;          // g_params in device memory: stub->req is where the batch's requests start in the ring
  uint32_t req_bytes;        // bytes per request (a multiple of 16); requests are contiguous in the ring window
  uint32_t batch, max_batch; // rows past `batch` are zeroed up to max_batch
  uint32_t command;
  uint8_t* dst[TP_MAX_RANKS];       // dst[r]: rank r's input buffer [max_batch, req_bytes]
  uint32_t* ctrl[TP_MAX_RANKS];     // ctrl[r]: rank r's control record {command, batch}
  uint32_t* doorbell[TP_MAX_RANKS]; // doorbell[r]: rank r's sequence word
  uint32_t* seq;             // this rank's counter: every launch publishes ++*seq
  uint32_t* arrivals;        // zeroed word (block arrival counter)
};
cudaError_t srpc_tp_fanout(const TpFanout& f, cudaStream_t stream);

// Bound (ns) of the flag waits of the tensor-parallel kernels on the current device (default 2 s).  A wait that runs
// out sets GEMM_ERR_TP_SRC_WAIT in the status word and the kernel returns; nothing traps or spins on.
cudaError_t srpc_tp_set_wait_ns(uint64_t ns);
