// Pooled miss fetch for expert-parallel ranks on one node: a missing expert is not pulled through
// its owner's host link alone, every rank pulls 1/G of the record through ITS link and the pieces
// meet at the owner over NVLink. A layer call ends when the rank with the most misses has its
// experts, so what bounds it is the largest per-rank miss count times one link; with the pool it
// is the total miss bytes over all G links. (No counterpart in the reference, which is single-GPU:
// src/cpp_worker/model_loader.cpp:75-79. The cache decisions are untouched: only the route the
// bytes of a demand copy take changes.)
//
// What is needed for that, all of it here:
//   * the pinned expert records of every rank live in POSIX shared memory that every rank maps and
//     registers with CUDA, so any rank can DMA any expert's bytes (rt_pin_all with a shared prefix,
//     rt_pool_open_peer);
//   * a mailbox in shared memory through which the ranks tell each other, per layer call, which
//     experts they miss (host to host, no device work; bounded waits);
//   * staging: each rank copies its slice of every missing record into one send buffer, grouped
//     by owner, and reports the split sizes of the all-to-all that follows (the collective itself
//     is the caller's: NCCL through torch.distributed);
//   * scatter: the owner moves the G slices of each of its records from the receive buffer into
//     the cache line and records the line's ready event.
#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstring>

#include "runtime.hpp"

namespace pm {

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Mail {
  int64_t seq;
  int32_t n;
  int32_t expert[kPoolMaxMiss];
};
constexpr int kMailSlots = 4;  // a rank is never more than one exchange ahead of another; four for margin

void* map_shared(const std::string& name, size_t bytes, bool create, std::string* err) {
  int fd = shm_open(name.c_str(), create ? (O_CREAT | O_RDWR) : O_RDWR, 0600);
  if (fd < 0) {
    *err = "shm_open(" + name + ") failed: " + std::strerror(errno);
    return nullptr;
  }
  if (create && ftruncate(fd, (off_t)bytes) != 0) {
    *err = "ftruncate(" + name + ") failed: " + std::strerror(errno);
    close(fd);
    return nullptr;
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) {
    *err = "mmap(" + name + ") failed: " + std::strerror(errno);
    return nullptr;
  }
  return p;
}

struct ScatterArgs {
  const unsigned char* src_base[64];  // start of source rank r's part of the receive buffer
  int32_t src_len[64];                // bytes of r's slice of one record
  unsigned char* line[kPoolMaxMiss];  // destination cache lines, in miss order
  size_t slice_bytes;                 // offset of slice r inside a record = r * slice_bytes
  int32_t n_ranks, n_miss;
};

// One CTA column per (miss, source): copies that slice from the receive buffer into its line.
__global__ void __launch_bounds__(256)
pool_scatter_kernel(const __grid_constant__ ScatterArgs a) {
  const int pair = blockIdx.x, m = pair / a.n_ranks, r = pair - m * a.n_ranks;
  const int len = a.src_len[r];
  const uint4* src = reinterpret_cast<const uint4*>(a.src_base[r] + (size_t)m * len);
  uint4* dst = reinterpret_cast<uint4*>(a.line[m] + (size_t)r * a.slice_bytes);
  const int n_vec = len / 16;
  for (int v = blockIdx.y * blockDim.x + threadIdx.x; v < n_vec; v += gridDim.y * blockDim.x) dst[v] = src[v];
}

}  // namespace

void* rt_shared_block(pm_ctx* c, const std::string& name, size_t bytes, bool create, std::string* err) {
  void* p = map_shared(name, bytes, create, err);
  if (p == nullptr) return nullptr;
  cudaError_t e = cudaHostRegister(p, bytes, cudaHostRegisterPortable);
  if (e != cudaSuccess) {
    *err = std::string("cudaHostRegister(") + name + "): " + cudaGetErrorString(e);
    munmap(p, bytes);
    return nullptr;
  }
  c->shared_blocks.push_back({p, bytes, create ? name : std::string()});
  return p;
}

void rt_release_shared_blocks(pm_ctx* c) {
  for (auto& b : c->shared_blocks) {
    cudaHostUnregister(b.ptr);
    munmap(b.ptr, b.bytes);
    if (!b.unlink_name.empty()) shm_unlink(b.unlink_name.c_str());
  }
  c->shared_blocks.clear();
  if (c->pool_mail != nullptr) {
    munmap(c->pool_mail, c->pool_mail_bytes);
    c->pool_mail = nullptr;
    if (c->pool_rank == 0 && !c->pool_mail_name.empty()) shm_unlink(c->pool_mail_name.c_str());
  }
}

int rt_pool_init(pm_ctx* c, int rank, int world, const char* mailbox_name) {
  if (world <= 0 || world > 64 || rank < 0 || rank >= world) return fail(PM_ERR_INVALID, "pool_init: bad rank or world size");
  if (!c->pinned || c->shared_prefix.empty())
    return fail(PM_ERR_STATE, "pool_init needs pin_all with a shared arena (context option shared_arena)");
  if (c->pool_mail != nullptr) return fail(PM_ERR_STATE, "pool_init called twice");
  std::string err;
  c->pool_mail_bytes = sizeof(Mail) * kMailSlots * (size_t)world;
  void* p = map_shared(mailbox_name, c->pool_mail_bytes, true, &err);  // every rank creates-or-opens: zero-filled by the kernel
  if (p == nullptr) return fail(PM_ERR_STATE, err);
  c->pool_mail = p;
  c->pool_mail_name = mailbox_name;
  c->pool_rank = rank;
  c->pool_world = world;
  c->peer_arena.assign(world, {});
  c->peer_num_expert.assign(world, 0);
  c->peer_arena[rank] = c->arena_blocks;
  c->peer_num_expert[rank] = c->cfg.num_expert;
  const size_t rec = c->param_offset.back();
  c->pool_slice = align_up((rec + world - 1) / world, 256);
  return PM_OK;
}

int rt_pool_open_peer(pm_ctx* c, int peer, const char* prefix, int peer_num_expert) {
  if (c->pool_mail == nullptr) return fail(PM_ERR_STATE, "pool_open_peer before pool_init");
  if (peer < 0 || peer >= c->pool_world || peer == c->pool_rank || peer_num_expert <= 0)
    return fail(PM_ERR_INVALID, "pool_open_peer: bad peer");
  const size_t rec = c->param_offset.back();
  std::vector<void*> blocks;
  for (int l = 0; l < c->cfg.num_layer; ++l) {
    std::string err;
    void* p = rt_shared_block(c, std::string(prefix) + "_L" + std::to_string(l), rec * (size_t)peer_num_expert, false, &err);
    if (p == nullptr) return fail(PM_ERR_STATE, err);
    blocks.push_back(p);
  }
  c->peer_arena[peer] = blocks;
  c->peer_num_expert[peer] = peer_num_expert;
  return PM_OK;
}

// Posts this rank's miss list for exchange `seq` and collects every rank's. out: [world][1 + kPoolMaxMiss]
// (count, then expert ids). Waits at most `timeout_s` for each peer.
int rt_pool_exchange(pm_ctx* c, int64_t seq, const int32_t* experts, int n, int32_t* out, double timeout_s) {
  if (c->pool_mail == nullptr) return fail(PM_ERR_STATE, "pool_exchange before pool_init");
  if (n < 0 || n > kPoolMaxMiss || seq <= 0) return fail(PM_ERR_INVALID, "pool_exchange: bad list");
  Mail* mail = static_cast<Mail*>(c->pool_mail);
  const int slot = (int)(seq % kMailSlots);
  Mail& mine = mail[(size_t)c->pool_rank * kMailSlots + slot];
  mine.n = n;
  for (int i = 0; i < n; ++i) mine.expert[i] = experts[i];
  std::atomic_thread_fence(std::memory_order_release);
  reinterpret_cast<std::atomic<int64_t>*>(&mine.seq)->store(seq, std::memory_order_release);
  const auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; r < c->pool_world; ++r) {
    Mail& m = mail[(size_t)r * kMailSlots + slot];
    while (reinterpret_cast<std::atomic<int64_t>*>(&m.seq)->load(std::memory_order_acquire) != seq) {
      if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s)
        return fail(PM_ERR_TIMEOUT, "pool_exchange: rank " + std::to_string(r) + " did not post its miss list in time");
    }
    int32_t* row = out + (size_t)r * (1 + kPoolMaxMiss);
    row[0] = m.n;
    for (int i = 0; i < m.n && i < kPoolMaxMiss; ++i) row[1 + i] = m.expert[i];
  }
  return PM_OK;
}

// Copies this rank's slice of every missing record of every owner into send_dev (grouped by owner,
// in list order) on `s`, and fills the byte counts of the all-to-all: send_split[o] to owner o,
// recv_split[r] from source r (this rank's misses times r's slice length).
int rt_pool_stage(pm_ctx* c, int layer, const int32_t* lists, void* send_dev, size_t send_cap, size_t recv_cap,
                  int64_t* send_split, int64_t* recv_split, cudaStream_t s) {
  if (c->pool_mail == nullptr) return fail(PM_ERR_STATE, "pool_stage before pool_init");
  if (layer < 0 || layer >= c->cfg.num_layer) return fail(PM_ERR_INVALID, "layer out of range");
  const int G = c->pool_world, me = c->pool_rank;
  const size_t rec = c->param_offset.back(), slice = c->pool_slice;
  auto len_of = [&](int r) -> size_t {
    const size_t b = (size_t)r * slice;
    return b >= rec ? 0 : std::min(slice, rec - b);
  };
  const size_t my_len = len_of(me), my_off = (size_t)me * slice;
  size_t send_total = 0, recv_total = 0;
  const int n_mine = lists[(size_t)me * (1 + kPoolMaxMiss)];
  for (int o = 0; o < G; ++o) {
    send_split[o] = (int64_t)lists[(size_t)o * (1 + kPoolMaxMiss)] * (int64_t)my_len;
    recv_split[o] = (int64_t)n_mine * (int64_t)len_of(o);
    send_total += (size_t)send_split[o];
    recv_total += (size_t)recv_split[o];
  }
  if (send_total > send_cap || recv_total > recv_cap)
    return fail(PM_ERR_INVALID, "pool_stage: the exchange buffers are too small for this many misses");
  unsigned char* dst = static_cast<unsigned char*>(send_dev);
  for (int o = 0; o < G; ++o) {
    const int32_t* row = lists + (size_t)o * (1 + kPoolMaxMiss);
    if (row[0] > 0 && (c->peer_arena[o].empty() || c->peer_num_expert[o] <= 0))
      return fail(PM_ERR_STATE, "pool_stage: the arena of rank " + std::to_string(o) + " was not opened");
    for (int i = 0; i < row[0]; ++i) {
      const int e = row[1 + i];
      if (e < 0 || e >= c->peer_num_expert[o]) return fail(PM_ERR_INVALID, "pool_stage: expert id out of range in a miss list");
      if (my_len > 0) {
        const unsigned char* src = static_cast<const unsigned char*>(c->peer_arena[o][layer]) + rec * (size_t)e + my_off;
        PM_CUDA(cudaMemcpyAsync(dst, src, my_len, cudaMemcpyHostToDevice, s));
        dst += my_len;
      }
    }
  }
  c->pool_bytes_pulled += (int64_t)send_total;
  return PM_OK;
}

// After the all-to-all: moves the slices of this rank's collected demand copies from recv_dev into
// their cache lines on `s` and records the lines' ready events.
int rt_pool_scatter(pm_ctx* c, const void* recv_dev, cudaStream_t s) {
  const std::vector<Action>& pooled = rt_pending_pooled(c);
  if (pooled.empty()) return PM_OK;
  if (c->pool_mail == nullptr) return fail(PM_ERR_STATE, "pool_scatter before pool_init");
  if (pooled.size() > (size_t)kPoolMaxMiss) return fail(PM_ERR_INVALID, "pool_scatter: too many collected copies");
  const int G = c->pool_world;
  const size_t rec = c->param_offset.back(), slice = c->pool_slice;
  ScatterArgs a{};
  a.n_ranks = G;
  a.n_miss = (int)pooled.size();
  a.slice_bytes = slice;
  size_t off = 0;
  for (int r = 0; r < G; ++r) {
    const size_t b = (size_t)r * slice;
    const size_t len = b >= rec ? 0 : std::min(slice, rec - b);
    a.src_base[r] = static_cast<const unsigned char*>(recv_dev) + off;
    a.src_len[r] = (int32_t)len;
    off += len * pooled.size();
  }
  for (size_t m = 0; m < pooled.size(); ++m) {
    const int line = pooled[m].line;
    a.line[m] = c->slab + (size_t)line * c->line_stride;
    // the line may still be read by an earlier launch, or written by an earlier copy on another stream
    if (c->line_read[line] != nullptr) PM_CUDA(cudaStreamWaitEvent(s, c->line_read[line], 0));
    if (c->line_copy_stream[line] != nullptr && c->line_copy_stream[line] != s)
      PM_CUDA(cudaStreamWaitEvent(s, c->line_ready[line], 0));
    c->line_copy_stream[line] = s;
  }
  pool_scatter_kernel<<<dim3((unsigned)(pooled.size() * G), 8), 256, 0, s>>>(a);
  PM_CUDA(cudaGetLastError());
  c->kernel_launches += 1;
  for (const Action& p : pooled) {
    PM_CUDA(cudaEventRecord(c->line_ready[p.line], s));
    c->line_pending[p.line] = 1;
    c->line_waiter[p.line] = nullptr;
  }
  return PM_OK;
}

// Fallback for a layer call whose misses do not fit the exchange buffers: the collected copies
// are enqueued on this rank's own copy stream after all.
int rt_pool_fetch_locally(pm_ctx* c) {
  const std::vector<Action> pooled = rt_pending_pooled(c);
  const int N = c->cfg.num_per_expert_param();
  for (const Action& a : pooled) {
    c->h2d_bytes -= (int64_t)c->param_offset[N];  // enqueue_copy counts the copy again
    c->h2d_copies -= 1;
  }
  return rt_execute_copies(c, pooled);
}

}  // namespace pm
