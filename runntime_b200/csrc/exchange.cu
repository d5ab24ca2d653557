// Set-up of the cross-GPU exchange of decode partials behind the C ABI: every rank
// allocates one block (its exchange buffer, its control words and its staging rows),
// hands the others a handle to it, and maps theirs.  Two ways to meet a peer:
//   - another process (one process per GPU): CUDA IPC handles, 64 bytes each, carried by
//     whatever channel the host has (a pipe, a socket, a file);
//   - the same process (one process owning several devices): the peer's block is used
//     directly, with peer access enabled between the two devices.
// No collective library and no launcher is involved; the kernels only ever see plain
// device pointers (peer memory is written with ordinary stores, never through a multicast
// mapping).  The reference has no multi-device code; this serves the KV-sequence sharding
// of rt_attn_decode (rt_attn.h).
#include <cstring>
#include <string>

#include "common.cuh"

struct rt_xmem {
  uint32_t magic;
  int device;
  int world, rank, batch, qHeads, headDim;
  size_t partialBytes, controlBytes, stageBytes;
  char* base;                       // this rank's block
  char* peer[RT_MAX_PEERS];         // every rank's block as mapped here (peer[rank] == base)
  bool ipc[RT_MAX_PEERS];           // mapped with cudaIpcOpenMemHandle: to be closed
};

namespace {

constexpr uint32_t kXLive = 0x52545858u;  // 'RTXX'

int xfail(int code, const std::string& msg) {
  rt::set_thread_error(msg.c_str());
  return code;
}

size_t round256(size_t n) { return (n + 255) / 256 * 256; }

int xenter(rt_xmem* m) {
  if (!m || m->magic != kXLive) return xfail(RT_INVALID_ARGUMENT, "not an exchange-memory handle");
  cudaError_t e = cudaSetDevice(m->device);
  if (e != cudaSuccess)
    return xfail(RT_EXECUTION_FAILED, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  return RT_OK;
}

}  // namespace

extern "C" {

int rt_xmem_create(int device, int32_t world, int32_t rank, int32_t batch, int32_t qHeads,
                   int32_t headDim, rt_xmem** out) {
  if (!out) return xfail(RT_INVALID_ARGUMENT, "rt_xmem_create: out is NULL");
  *out = nullptr;
  if (world < 1 || world > RT_MAX_PEERS || rank < 0 || rank >= world)
    return xfail(RT_INVALID_ARGUMENT, "rt_xmem_create: world must be 1..8 and rank inside it");
  if (batch < world || qHeads < 1 || headDim < 1 || headDim > 128)
    return xfail(RT_INVALID_ARGUMENT,
                 "rt_xmem_create: batch must be at least world, qHeads and headDim (at most 128) positive");
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess)
    return xfail(RT_EXECUTION_FAILED, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  rt_xmem* m = new rt_xmem();
  m->magic = kXLive;
  m->device = device;
  m->world = world, m->rank = rank, m->batch = batch, m->qHeads = qHeads, m->headDim = headDim;
  const size_t row = (size_t)(2 + headDim) * sizeof(float);
  const size_t per = (size_t)rt::exchange_per(batch, world);
  m->partialBytes = round256(2 * (size_t)world * per * qHeads * row);
  m->controlBytes = round256((size_t)(2 * world + 3) * sizeof(uint32_t));
  m->stageBytes = round256((size_t)batch * qHeads * row);
  const size_t total = m->partialBytes + m->controlBytes + m->stageBytes;
  void* ptr = nullptr;
  if ((e = cudaMalloc(&ptr, total)) != cudaSuccess || (e = cudaMemset(ptr, 0, total)) != cudaSuccess ||
      (e = cudaDeviceSynchronize()) != cudaSuccess) {
    if (ptr) cudaFree(ptr);
    delete m;
    return xfail(RT_EXECUTION_FAILED, std::string("rt_xmem_create: ") + cudaGetErrorString(e));
  }
  m->base = static_cast<char*>(ptr);
  for (int r = 0; r < RT_MAX_PEERS; r++) m->peer[r] = nullptr, m->ipc[r] = false;
  m->peer[rank] = m->base;
  *out = m;
  return RT_OK;
}

int rt_xmem_export(rt_xmem* m, void* handle) {
  if (int s = xenter(m)) return s;
  if (!handle) return xfail(RT_INVALID_ARGUMENT, "rt_xmem_export: handle is NULL");
  static_assert(sizeof(cudaIpcMemHandle_t) == RT_XMEM_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, m->base);
  if (e != cudaSuccess)
    return xfail(RT_EXECUTION_FAILED, std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
  std::memcpy(handle, &h, sizeof h);
  return RT_OK;
}

int rt_xmem_import(rt_xmem* m, int32_t peer, const void* handle) {
  if (int s = xenter(m)) return s;
  if (!handle || peer < 0 || peer >= m->world || peer == m->rank)
    return xfail(RT_INVALID_ARGUMENT, "rt_xmem_import: peer must be another rank of the world");
  if (m->peer[peer]) return xfail(RT_INVALID_ARGUMENT, "rt_xmem_import: that peer is already mapped");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof h);
  void* ptr = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess)
    return xfail(RT_EXECUTION_FAILED, std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
  m->peer[peer] = static_cast<char*>(ptr);
  m->ipc[peer] = true;
  return RT_OK;
}

int rt_xmem_attach(rt_xmem* m, int32_t peer, rt_xmem* other) {
  if (int s = xenter(m)) return s;
  if (!other || other->magic != kXLive || peer < 0 || peer >= m->world || peer == m->rank)
    return xfail(RT_INVALID_ARGUMENT, "rt_xmem_attach: peer must be another rank's live handle");
  if (other->rank != peer || other->world != m->world || other->batch != m->batch ||
      other->qHeads != m->qHeads || other->headDim != m->headDim)
    return xfail(RT_INVALID_ARGUMENT, "rt_xmem_attach: the peer's handle was made for another shape or rank");
  if (m->peer[peer]) return xfail(RT_INVALID_ARGUMENT, "rt_xmem_attach: that peer is already mapped");
  if (other->device != m->device) {
    int can = 0;
    cudaError_t e = cudaDeviceCanAccessPeer(&can, m->device, other->device);
    if (e != cudaSuccess || !can)
      return xfail(RT_UNSUPPORTED_DEVICE, "rt_xmem_attach: device " + std::to_string(m->device) +
                                              " cannot reach device " + std::to_string(other->device));
    e = cudaDeviceEnablePeerAccess(other->device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      cudaGetLastError();
    } else if (e != cudaSuccess) {
      return xfail(RT_EXECUTION_FAILED,
                   std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e));
    }
  }
  m->peer[peer] = other->base;
  return RT_OK;
}

int rt_xmem_exchange(rt_xmem* m, rt_exchange* out) {
  if (int s = xenter(m)) return s;
  if (!out) return xfail(RT_INVALID_ARGUMENT, "rt_xmem_exchange: out is NULL");
  std::memset(out, 0, sizeof *out);
  for (int r = 0; r < m->world; r++) {
    if (!m->peer[r])
      return xfail(RT_NOT_INITIALIZED,
                   "rt_xmem_exchange: rank " + std::to_string(r) + " has not been imported or attached");
    out->partials[r] = reinterpret_cast<float*>(m->peer[r]);
    out->flags[r] = reinterpret_cast<uint32_t*>(m->peer[r] + m->partialBytes);
  }
  out->world = m->world;
  out->rank = m->rank;
  out->step = reinterpret_cast<uint32_t*>(m->base + m->partialBytes) + m->world;
  out->stage = reinterpret_cast<float*>(m->base + m->partialBytes + m->controlBytes);
  out->phases = 0;
  return RT_OK;
}

int rt_xmem_destroy(rt_xmem* m) {
  if (int s = xenter(m)) return s;
  cudaDeviceSynchronize();
  for (int r = 0; r < m->world; r++)
    if (m->ipc[r] && m->peer[r]) cudaIpcCloseMemHandle(m->peer[r]);
  cudaFree(m->base);
  m->magic = 0;
  delete m;
  return RT_OK;
}

}  // extern "C"
