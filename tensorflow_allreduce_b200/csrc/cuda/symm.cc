#include "symm.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>
#include <unistd.h>

namespace bc {
namespace gpu {

namespace {

// Driver entry points are looked up at run time so that the library loads (and the CPU paths
// work) on machines without a GPU driver.
struct Driver {
  bool ok = false;
  std::string why;
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*memRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*memExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*memImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*memReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*memAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*memUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*memGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*mcCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*mcAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*mcBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*mcUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*mcGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*deviceGet)(CUdevice*, int) = nullptr;
  CUresult (*deviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*getErrorString)(CUresult, const char**) = nullptr;
};

template <typename F>
bool load(const char* name, F* fn, std::string* why) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    (void)cudaGetLastError();
    *why = std::string("driver entry point ") + name + " unavailable";
    return false;
  }
  *fn = reinterpret_cast<F>(p);
  return true;
}

Driver& driver() {
  static Driver d;
  static bool tried = false;
  if (tried) return d;
  tried = true;
  bool ok = true;
  ok = ok && load("cuMemCreate", &d.memCreate, &d.why);
  ok = ok && load("cuMemRelease", &d.memRelease, &d.why);
  ok = ok && load("cuMemExportToShareableHandle", &d.memExport, &d.why);
  ok = ok && load("cuMemImportFromShareableHandle", &d.memImport, &d.why);
  ok = ok && load("cuMemAddressReserve", &d.memReserve, &d.why);
  ok = ok && load("cuMemAddressFree", &d.memAddressFree, &d.why);
  ok = ok && load("cuMemMap", &d.memMap, &d.why);
  ok = ok && load("cuMemUnmap", &d.memUnmap, &d.why);
  ok = ok && load("cuMemSetAccess", &d.memSetAccess, &d.why);
  ok = ok && load("cuMemGetAllocationGranularity", &d.memGranularity, &d.why);
  ok = ok && load("cuDeviceGet", &d.deviceGet, &d.why);
  ok = ok && load("cuDeviceGetAttribute", &d.deviceGetAttribute, &d.why);
  ok = ok && load("cuGetErrorString", &d.getErrorString, &d.why);
  d.ok = ok;
  if (ok) {
    std::string w;
    bool mc = load("cuMulticastCreate", &d.mcCreate, &w) && load("cuMulticastAddDevice", &d.mcAddDevice, &w) &&
              load("cuMulticastBindMem", &d.mcBindMem, &w) && load("cuMulticastUnbind", &d.mcUnbind, &w) &&
              load("cuMulticastGetGranularity", &d.mcGranularity, &w);
    if (!mc) d.mcCreate = nullptr;
  }
  return d;
}

std::string cu_err(CUresult r) {
  const char* s = nullptr;
  if (driver().getErrorString && driver().getErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "CUresult " + std::to_string((int)r);
}

#define CUDA_RT(expr)                                                                            \
  do {                                                                                           \
    cudaError_t _e = (expr);                                                                     \
    if (_e != cudaSuccess) throw ::bc::Error(std::string(#expr) + ": " + cudaGetErrorString(_e)); \
  } while (0)

size_t round_up(size_t v, size_t g) { return (v + g - 1) / g * g; }

// All ranks learn whether every rank succeeded at a step; the first failure message wins.
bool all_ok(const HostAllgather& ag, bool mine, const std::string& my_msg, std::string* why) {
  std::string blob = mine ? std::string("1") : std::string("0") + my_msg;
  std::vector<std::string> all = ag(blob);
  bool ok = true;
  for (size_t r = 0; r < all.size(); r++) {
    if (all[r].empty() || all[r][0] != '1') {
      if (ok && why) *why = "rank " + std::to_string(r) + ": " + (all[r].size() > 1 ? all[r].substr(1) : std::string("failed"));
      ok = false;
    }
  }
  return ok;
}

}  // namespace

SymmAllocator::SymmAllocator(int rank, int world, int device, uint64_t job_id, Mode mode, bool want_multicast, double timeout_s)
    : rank_(rank), world_(world), device_(device), job_id_(job_id), want_mc_(want_multicast), mode_(mode), timeout_s_(timeout_s) {
  BC_CHECK(world <= dev::kMaxRanks, "at most " << dev::kMaxRanks << " ranks per node are supported, got " << world);
  CUDA_RT(cudaSetDevice(device));
  CUDA_RT(cudaFree(0));
  if (world > 1) {
    char name[128];
    snprintf(name, sizeof(name), "bcoll-%016llx-fd-%d", (unsigned long long)job_id, rank);
    fd_listener_ = Socket::listen_unix(name, world + 4);
  }
}

SymmAllocator::~SymmAllocator() { release_all(); }

std::string SymmAllocator::describe() const {
  std::string s = use_vmm_ ? "vmm" : "ipc";
  if (mc_ok_) s += "+multicast";
  return s;
}

Segment* SymmAllocator::find(const void* p, size_t bytes) const {
  const char* c = (const char*)p;
  for (const auto& s : segs_)
    if (c >= s->local && c + bytes <= s->local + s->size) return s.get();
  return nullptr;
}

bool SymmAllocator::alloc_vmm(Segment* s, size_t bytes, const HostAllgather& ag, std::string* why) {
  Driver& d = driver();
  std::string msg;
  bool ok = d.ok;
  if (!ok) msg = d.why;

  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;

  size_t gran = 2u << 20;
  CUmemGenericAllocationHandle h = 0;
  int fd = -1;
  size_t size = bytes;
  if (ok) {
    CUresult r = d.memGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (r != CUDA_SUCCESS) { ok = false; msg = "cuMemGetAllocationGranularity: " + cu_err(r); }
  }
  if (ok && want_mc_ && d.mcCreate && world_ > 1) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = world_;
    mp.size = round_up(bytes, gran);
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d.mcGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
  }
  if (ok) {
    size = round_up(bytes, gran);
    CUresult r = d.memCreate(&h, size, &prop, 0);
    if (r != CUDA_SUCCESS) { ok = false; msg = "cuMemCreate(" + std::to_string(size) + "): " + cu_err(r); }
  }
  if (ok && world_ > 1) {
    CUresult r = d.memExport(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) { ok = false; msg = "cuMemExportToShareableHandle: " + cu_err(r); }
  }
  if (!all_ok(ag, ok, msg, why)) {
    if (fd >= 0) ::close(fd);
    if (h) d.memRelease(h);
    return false;
  }

  // Pass the descriptor to every peer and collect theirs.
  std::vector<int> fds(world_, -1);
  const double deadline = now_s() + timeout_s_;
  try {
    for (int k = 1; k < world_; k++) {
      const int p = (rank_ + k) % world_;
      char name[128];
      snprintf(name, sizeof(name), "bcoll-%016llx-fd-%d", (unsigned long long)job_id_, p);
      Socket c = Socket::connect_unix(name, deadline);
      c.send_fd(fd, (int32_t)((s->id << 8) | rank_), deadline);
      // the descriptor stays queued in the peer's socket after this end closes
    }
    for (int k = 1; k < world_; k++) {
      Socket c = fd_listener_.accept(deadline);
      int32_t tag = 0;
      int got = c.recv_fd(&tag, deadline);
      const int from = tag & 0xff;
      if ((tag >> 8) != s->id || from < 0 || from >= world_ || from == rank_ || fds[from] >= 0) {
        ::close(got);
        throw Error("unexpected descriptor tag while exchanging symmetric memory handles");
      }
      fds[from] = got;
    }
  } catch (const std::exception& e) {
    ok = false;
    msg = e.what();
  }
  if (fd >= 0) ::close(fd);

  // Import and map.
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int p = 0; p < world_ && ok; p++) {
    CUmemGenericAllocationHandle ph = h;
    if (p != rank_) {
      CUresult r = d.memImport(&ph, (void*)(uintptr_t)fds[p], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (r != CUDA_SUCCESS) { ok = false; msg = "cuMemImportFromShareableHandle: " + cu_err(r); break; }
    }
    s->handles[p] = ph;
    CUdeviceptr va = 0;
    CUresult r = d.memReserve(&va, size, gran, 0, 0);
    if (r == CUDA_SUCCESS) r = d.memMap(va, size, 0, ph, 0);
    if (r == CUDA_SUCCESS) r = d.memSetAccess(va, size, &acc, 1);
    if (r != CUDA_SUCCESS) { ok = false; msg = "mapping peer " + std::to_string(p) + ": " + cu_err(r); break; }
    s->peer[p] = (char*)va;
  }
  for (int p = 0; p < world_; p++)
    if (fds[p] >= 0) ::close(fds[p]);
  if (!all_ok(ag, ok, msg, why)) return false;
  s->local = s->peer[rank_];
  s->size = size;
  s->vmm = true;
  return true;
}

bool SymmAllocator::bind_multicast(Segment* s, const HostAllgather& ag, std::string* why) {
  Driver& d = driver();
  std::string msg;
  bool ok = d.mcCreate != nullptr;
  if (!ok) msg = "multicast entry points unavailable";
  CUdevice cudev = 0;
  if (ok) {
    int sup = 0;
    if (d.deviceGet(&cudev, device_) != CUDA_SUCCESS ||
        d.deviceGetAttribute(&sup, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev) != CUDA_SUCCESS || !sup) {
      ok = false;
      msg = "device does not support multicast";
    }
  }
  if (!all_ok(ag, ok, msg, why)) return false;

  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = world_;
  mp.size = s->size;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle mch = 0;
  int fd = -1;
  const double deadline = now_s() + timeout_s_;
  if (rank_ == 0) {
    CUresult r = d.mcCreate(&mch, &mp);
    if (r != CUDA_SUCCESS) { ok = false; msg = "cuMulticastCreate: " + cu_err(r); }
    if (ok) {
      r = d.memExport(&fd, mch, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) { ok = false; msg = "export multicast handle: " + cu_err(r); }
    }
  }
  if (!all_ok(ag, ok, msg, why)) {
    if (mch) d.memRelease(mch);
    return false;
  }
  try {
    if (rank_ == 0) {
      for (int p = 1; p < world_; p++) {
        char name[128];
        snprintf(name, sizeof(name), "bcoll-%016llx-fd-%d", (unsigned long long)job_id_, p);
        Socket c = Socket::connect_unix(name, deadline);
        c.send_fd(fd, (int32_t)((s->id << 8) | 0xfe), deadline);
      }
      ::close(fd);
    } else {
      Socket c = fd_listener_.accept(deadline);
      int32_t tag = 0;
      int got = c.recv_fd(&tag, deadline);
      CUresult r = d.memImport(&mch, (void*)(uintptr_t)got, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      ::close(got);
      if (r != CUDA_SUCCESS) { ok = false; msg = "import multicast handle: " + cu_err(r); }
    }
  } catch (const std::exception& e) {
    ok = false;
    msg = e.what();
  }
  if (ok) {
    CUresult r = d.mcAddDevice(mch, cudev);
    if (r != CUDA_SUCCESS) { ok = false; msg = "cuMulticastAddDevice: " + cu_err(r); }
  }
  // Every device must have been added before any memory is bound.
  if (!all_ok(ag, ok, msg, why)) {
    if (mch) d.memRelease(mch);
    return false;
  }
  {
    CUresult r = d.mcBindMem(mch, 0, s->handles[rank_], 0, s->size, 0);
    if (r != CUDA_SUCCESS) { ok = false; msg = "cuMulticastBindMem: " + cu_err(r); }
  }
  CUdeviceptr va = 0;
  if (ok) {
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device_;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CUresult r = d.memReserve(&va, s->size, 0, 0, 0);
    if (r == CUDA_SUCCESS) r = d.memMap(va, s->size, 0, mch, 0);
    if (r == CUDA_SUCCESS) r = d.memSetAccess(va, s->size, &acc, 1);
    if (r != CUDA_SUCCESS) { ok = false; msg = "mapping multicast object: " + cu_err(r); }
  }
  s->mc_handle = mch;
  s->mc_size = s->size;
  if (!all_ok(ag, ok, msg, why)) {
    // Leave the object bound but unused; it is released with the segment.
    s->mc = nullptr;
    return false;
  }
  s->mc = (char*)va;
  return true;
}

void SymmAllocator::alloc_ipc(Segment* s, size_t bytes, const HostAllgather& ag) {
  const size_t size = round_up(bytes, 2u << 20);
  void* p = nullptr;
  std::string msg;
  bool ok = true;
  cudaError_t e = cudaMalloc(&p, size);
  if (e != cudaSuccess) { ok = false; msg = std::string("cudaMalloc: ") + cudaGetErrorString(e); }
  cudaIpcMemHandle_t mh;
  memset(&mh, 0, sizeof(mh));
  if (ok && world_ > 1) {
    e = cudaIpcGetMemHandle(&mh, p);
    if (e != cudaSuccess) { ok = false; msg = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e); }
  }
  std::string why;
  if (!all_ok(ag, ok, msg, &why)) {
    if (p) cudaFree(p);
    throw Error("symmetric allocation failed: " + why);
  }
  std::vector<std::string> all = ag(std::string((const char*)&mh, sizeof(mh)));
  s->peer[rank_] = (char*)p;
  for (int q = 0; q < world_ && ok; q++) {
    if (q == rank_) continue;
    cudaIpcMemHandle_t ph;
    memcpy(&ph, all[q].data(), sizeof(ph));
    void* pp = nullptr;
    e = cudaIpcOpenMemHandle(&pp, ph, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { ok = false; msg = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e); break; }
    s->peer[q] = (char*)pp;
  }
  if (!all_ok(ag, ok, msg, &why)) throw Error("symmetric allocation failed: " + why);
  s->local = (char*)p;
  s->size = size;
  s->vmm = false;
}

Segment* SymmAllocator::alloc(size_t bytes, const HostAllgather& ag) {
  CUDA_RT(cudaSetDevice(device_));
  std::unique_ptr<Segment> s(new Segment());
  s->id = (int)segs_.size();
  if (!decided_) {
    decided_ = true;
    use_vmm_ = (mode_ != Mode::IPC);
  }
  if (use_vmm_) {
    std::string why;
    if (!alloc_vmm(s.get(), bytes, ag, &why)) {
      BC_CHECK(mode_ != Mode::VMM && segs_.empty(), "symmetric allocation (VMM) failed: " << why);
      BC_LOG(1, "VMM symmetric memory unavailable (%s); using CUDA IPC", why.c_str());
      use_vmm_ = false;
      *s = Segment();
      s->id = (int)segs_.size();
    }
  }
  if (!use_vmm_) alloc_ipc(s.get(), bytes, ag);
  CUDA_RT(cudaMemset(s->local, 0, s->size));
  CUDA_RT(cudaDeviceSynchronize());
  if (use_vmm_ && want_mc_ && world_ > 1 && (segs_.empty() || mc_ok_)) {
    std::string why;
    mc_ok_ = bind_multicast(s.get(), ag, &why);
    if (!mc_ok_) BC_LOG(1, "NVLS multicast not used: %s", why.c_str());
  }
  ag(std::string());  // everyone has mapped and cleared before anyone touches peer memory
  segs_.push_back(std::move(s));
  return segs_.back().get();
}

void SymmAllocator::release_all() {
  if (segs_.empty()) return;
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  Driver& d = driver();
  for (auto& s : segs_) {
    if (s->vmm) {
      if (s->mc) {
        d.memUnmap((CUdeviceptr)s->mc, s->mc_size);
        d.memAddressFree((CUdeviceptr)s->mc, s->mc_size);
      }
      if (s->mc_handle) {
        CUdevice cudev = 0;
        if (d.deviceGet(&cudev, device_) == CUDA_SUCCESS) d.mcUnbind(s->mc_handle, cudev, 0, s->mc_size);
        d.memRelease(s->mc_handle);
      }
      for (int p = 0; p < world_; p++) {
        if (s->peer[p]) {
          d.memUnmap((CUdeviceptr)s->peer[p], s->size);
          d.memAddressFree((CUdeviceptr)s->peer[p], s->size);
        }
        if (s->handles[p]) d.memRelease(s->handles[p]);
      }
    } else {
      for (int p = 0; p < world_; p++) {
        if (p != rank_ && s->peer[p]) cudaIpcCloseMemHandle(s->peer[p]);
      }
      if (s->local) cudaFree(s->local);
    }
  }
  segs_.clear();
}

}  // namespace gpu
}  // namespace bc
