// Host side of the streaming sampler (stream.cuh): launch helpers shared by the sampler and the verifier, and the
// C-ABI entry points of the vocabulary-sharded path (a shard publishes the records of its chunks, the caller
// all-gathers them, every rank combines).
#include "ds41_b200.h"
#include "host_error.h"
#include "stream.cuh"
#include <cmath>

namespace ds41 {

static_assert(sizeof(ChunkRecord) == sizeof(ds41_b200_shard_row), "shard record layout");

int chunks_for(int vocab) { return (vocab + kChunkIds - 1) / kChunkIds; }

cudaError_t launch_chunks(const ChunkArgs &a, int rows, cudaStream_t stream) {
  chunk_kernel<<<unsigned(rows) * unsigned(a.chunks), kChunkThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_combine(const CombineArgs &a, bool stats, cudaStream_t stream) {
  static thread_local int configured = -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (configured != dev) {  // the combine needs more than the default 48 KB of dynamic shared memory
    e = cudaFuncSetAttribute(combine_kernel<kCombineStats>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(CombineSmem)));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(combine_kernel<kCombineDraw>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(CombineSmem)));
    if (e != cudaSuccess) return e;
    configured = dev;
  }
  if (stats) combine_kernel<kCombineStats><<<a.rows, kCombineThreads, sizeof(CombineSmem), stream>>>(a);
  else combine_kernel<kCombineDraw><<<a.rows, kCombineThreads, sizeof(CombineSmem), stream>>>(a);
  return cudaGetLastError();
}

}  // namespace ds41

using namespace ds41;

extern "C" int ds41_b200_shard_chunks(int vocab_local) { return vocab_local < 1 ? 0 : chunks_for(vocab_local); }

extern "C" int ds41_b200_shard_candidates(const ds41_b200_shard_args *p, cudaStream_t stream) {
  if (!p || p->struct_bytes != sizeof(ds41_b200_shard_args)) return invalid("shard args: struct size / ABI mismatch");
  if (p->rows < 1 || p->vocab_local < 1 || p->vocab_offset < 0 || !p->logits || p->logits_stride < p->vocab_local || !p->out)
    return invalid("shard arguments");
  const int chunks = p->chunks > 0 ? p->chunks : chunks_for(p->vocab_local);
  if (chunks < chunks_for(p->vocab_local)) return invalid("shard arguments: too few chunks for the local vocabulary");
  if (!std::isfinite(p->temperature) || p->temperature < 0) return invalid("temperature/top_p/logits");
  ChunkArgs a{p->logits, p->logits_stride, p->vocab_local, p->vocab_offset, chunks,
              p->temperature > 0 ? std::fmax(p->temperature, 1e-5) : 0.0, reinterpret_cast<ChunkRecord *>(p->out)};
  return int(launch_chunks(a, p->rows, stream));
}

extern "C" int ds41_b200_shard_combine(const ds41_b200_shard_combine_args *p, cudaStream_t stream) {
  if (!p || p->struct_bytes != sizeof(ds41_b200_shard_combine_args)) return invalid("combine args: struct size / ABI mismatch");
  if (p->rows < 1 || p->ranks < 1 || p->chunks < 1 || p->ranks * p->chunks > kMaxRecords || p->vocab < 1 || !p->gathered ||
      !p->seeds || !p->steps || !p->tokens)
    return invalid("combine arguments (at most 17 chunk records per row)");
  if (!std::isfinite(p->temperature) || p->temperature < 0 || !std::isfinite(p->top_p) || p->top_p <= 0 || p->top_p > 1 || p->top_k < 0)
    return invalid("temperature/top_p/logits");
  if (p->slot > 5 || p->purpose > 3) return invalid("Philox v2 address out of range");
  CombineArgs a{reinterpret_cast<const ChunkRecord *>(p->gathered), p->rows, p->ranks, p->chunks, p->vocab,
                p->temperature > 0 ? std::fmax(p->temperature, 1e-5) : 0.0, p->top_p, p->top_k, p->seeds, p->steps, p->slot,
                p->purpose, p->tokens, p->status, nullptr};
  return int(launch_combine(a, false, stream));
}
