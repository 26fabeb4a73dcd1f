#include "symm_arena.h"

#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <map>

#include <cuda_runtime_api.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include "../common/logging.h"
#include "cuda_driver.h"

namespace hvd {

namespace {

// ---- descriptor passing over abstract Unix-domain sockets -----------------

struct FdMessage {
  int32_t from_rank;
  int32_t tag;
};

socklen_t AbstractAddr(uint64_t token, int rank, sockaddr_un* addr) {
  std::memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  char name[96];
  int n = std::snprintf(name, sizeof(name), "hvdb200-%016llx-%d",
                        static_cast<unsigned long long>(token), rank);
  // Leading NUL selects the abstract namespace (no file system entry).
  std::memcpy(addr->sun_path + 1, name, static_cast<size_t>(n));
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

int MakeListener(uint64_t token, int rank) {
  int fd = socket(AF_UNIX, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  sockaddr_un addr;
  socklen_t len = AbstractAddr(token, rank, &addr);
  if (bind(fd, reinterpret_cast<sockaddr*>(&addr), len) != 0 ||
      listen(fd, 64) != 0) {
    close(fd);
    return -1;
  }
  return fd;
}

bool SendFd(uint64_t token, int to_rank, int from_rank, int tag, int payload) {
  int s = socket(AF_UNIX, SOCK_STREAM, 0);
  if (s < 0) return false;
  sockaddr_un addr;
  socklen_t len = AbstractAddr(token, to_rank, &addr);
  bool ok = false;
  for (int attempt = 0; attempt < 200 && !ok; ++attempt) {
    if (connect(s, reinterpret_cast<sockaddr*>(&addr), len) == 0) ok = true;
    else usleep(10000);
  }
  if (ok) {
    FdMessage m = {from_rank, tag};
    struct iovec iov = {&m, sizeof(m)};
    char ctrl[CMSG_SPACE(sizeof(int))];
    std::memset(ctrl, 0, sizeof(ctrl));
    struct msghdr msg;
    std::memset(&msg, 0, sizeof(msg));
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &payload, sizeof(int));
    ok = sendmsg(s, &msg, MSG_NOSIGNAL) == static_cast<ssize_t>(sizeof(m));
  }
  close(s);
  return ok;
}

bool RecvFd(int listener, double timeout_s, FdMessage* m, int* payload) {
  struct pollfd pf = {listener, POLLIN, 0};
  if (poll(&pf, 1, static_cast<int>(timeout_s * 1000)) <= 0) return false;
  int s = accept(listener, nullptr, nullptr);
  if (s < 0) return false;
  struct iovec iov = {m, sizeof(*m)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  struct msghdr msg;
  std::memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  struct pollfd ps = {s, POLLIN, 0};
  bool ok = poll(&ps, 1, static_cast<int>(timeout_s * 1000)) > 0 &&
            recvmsg(s, &msg, 0) == static_cast<ssize_t>(sizeof(*m));
  if (ok) {
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    ok = c != nullptr && c->cmsg_level == SOL_SOCKET &&
         c->cmsg_type == SCM_RIGHTS;
    if (ok) std::memcpy(payload, CMSG_DATA(c), sizeof(int));
  }
  close(s);
  return ok;
}

// True only if every rank passes true.
bool Agree(Comm& comm, bool ok) {
  uint64_t w = ok ? ~0ull : 0ull;
  comm.AllreduceBits(&w, 1, true);
  return w == ~0ull;
}

}  // namespace

Status SymmArena::Create(Comm& comm, int device, size_t data_bytes,
                         bool want_multicast, uint64_t token) {
  Destroy();
  const int world = comm.size(), rank = comm.rank();
  if (world > SYMM_MAX_RANKS)
    return Status::PreconditionError("symmetric memory supports at most " +
                                     std::to_string(SYMM_MAX_RANKS) + " ranks");
  std::string err;
  const DriverApi* api = GetDriverApi(&err);
  bool ok = api != nullptr;
  CUdevice cudev = 0;
  int mc_supported = 0;
  if (ok) {
    ok = cudaSetDevice(device) == cudaSuccess &&
         cudaFree(nullptr) == cudaSuccess &&  // make sure the context exists
         api->DeviceGet(&cudev, device) == CUDA_SUCCESS;
    int vmm = 0, posix_fd = 0;
    if (ok) {
      api->DeviceGetAttribute(
          &vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, cudev);
      api->DeviceGetAttribute(
          &posix_fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED,
          cudev);
      if (api->MulticastCreate != nullptr)
        api->DeviceGetAttribute(&mc_supported,
                                CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev);
      ok = vmm && posix_fd;
      if (!ok) err = "device lacks VMM or POSIX-fd shareable handles";
    } else if (err.empty()) {
      err = "cannot select CUDA device " + std::to_string(device);
    }
  }
  if (!Agree(comm, ok))
    return Status::PreconditionError("symmetric memory unavailable: " +
                                     (err.empty() ? "a peer reported failure" : err));
  bool use_mc = Agree(comm, want_multicast && mc_supported != 0 && world > 1);

  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  CUresult r = api->MemGetAllocationGranularity(
      &gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS || gran == 0) gran = 2u << 20;
  CUmulticastObjectProp mc_prop;
  std::memset(&mc_prop, 0, sizeof(mc_prop));
  if (use_mc) {
    mc_prop.numDevices = static_cast<unsigned>(world);
    mc_prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mc_prop.size = gran;
    size_t mc_gran = 0;
    if (api->MulticastGetGranularity(&mc_gran, &mc_prop,
                                     CU_MULTICAST_GRANULARITY_RECOMMENDED) ==
            CUDA_SUCCESS && mc_gran > gran)
      gran = mc_gran;
  }
  const size_t signal_bytes = static_cast<size_t>(SYMM_FLAG_SETS) *
                              SYMM_FLAG_BANKS * SYMM_MAX_RANKS *
                              SYMM_MAX_BLOCKS * sizeof(uint32_t);
  const size_t data_rounded = static_cast<size_t>(RoundUp(data_bytes, 4096));
  total_bytes_ = static_cast<size_t>(RoundUp(data_rounded + signal_bytes, gran));

  // 1. allocate and export
  handles_.assign(world, 0);
  vas_.assign(world, 0);
  CUmemGenericAllocationHandle mine = 0;
  int my_fd = -1;
  r = api->MemCreate(&mine, total_bytes_, &prop, 0);
  ok = r == CUDA_SUCCESS;
  if (ok) {
    handles_[rank] = mine;
    r = api->MemExportToShareableHandle(&my_fd, mine,
                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    ok = r == CUDA_SUCCESS;
  }
  if (!ok) err = "cuMemCreate/export failed: " + DriverErrorString(api, r);
  int listener = ok ? MakeListener(token, rank) : -1;
  if (ok && listener < 0) {
    ok = false;
    err = "cannot create Unix socket for handle exchange";
  }
  if (!Agree(comm, ok)) {
    if (listener >= 0) close(listener);
    if (my_fd >= 0) close(my_fd);
    Destroy();
    return Status::PreconditionError("symmetric memory unavailable: " +
                                     (err.empty() ? "a peer reported failure" : err));
  }

  // 2. exchange descriptors (all listeners exist after the Agree above)
  for (int p = 0; p < world && ok; ++p)
    if (p != rank) ok = SendFd(token, p, rank, /*tag=*/1, my_fd);
  std::map<int, int> peer_fds;
  int mc_fd = -1;
  CUmemGenericAllocationHandle mc_handle = 0;
  if (use_mc && rank == 0 && ok) {
    mc_prop.size = total_bytes_;
    r = api->MulticastCreate(&mc_handle, &mc_prop);
    bool created = r == CUDA_SUCCESS;
    if (created) {
      r = api->MemExportToShareableHandle(
          &mc_fd, mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      created = r == CUDA_SUCCESS;
    }
    if (!created) {
      HVD_LOG(WARNING) << "NVLink multicast object could not be created ("
                       << DriverErrorString(api, r) << "); using peer loads/stores only";
      mc_fd = -1;
    }
    // Tag 2 carries the multicast descriptor, tag 3 says "no multicast"
    // (with a harmless descriptor so the message format stays the same).
    for (int p = 1; p < world && ok; ++p)
      ok = SendFd(token, p, 0, mc_fd >= 0 ? 2 : 3, mc_fd >= 0 ? mc_fd : my_fd);
  }
  int expected = (world - 1) + ((use_mc && rank != 0) ? 1 : 0);
  int mc_tag = 0;
  while (ok && expected > 0) {
    FdMessage m;
    int fd = -1;
    if (!RecvFd(listener, 60.0, &m, &fd)) {
      ok = false;
      err = "timed out receiving memory handles from peers";
      break;
    }
    if (m.tag == 1) peer_fds[m.from_rank] = fd;
    else {
      mc_tag = m.tag;
      if (m.tag == 2) mc_fd = fd; else close(fd);
    }
    --expected;
  }
  close(listener);

  // 3. import and map every rank's buffer
  CUmemAccessDesc access;
  std::memset(&access, 0, sizeof(access));
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int p = 0; p < world && ok; ++p) {
    if (p != rank) {
      CUmemGenericAllocationHandle h = 0;
      r = api->MemImportFromShareableHandle(
          &h, reinterpret_cast<void*>(static_cast<intptr_t>(peer_fds[p])),
          CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (r != CUDA_SUCCESS) {
        ok = false;
        err = "cuMemImportFromShareableHandle failed: " + DriverErrorString(api, r);
        break;
      }
      handles_[p] = h;
    }
    CUdeviceptr va = 0;
    r = api->MemAddressReserve(&va, total_bytes_, gran, 0, 0);
    if (r == CUDA_SUCCESS) {
      vas_[p] = va;
      r = api->MemMap(va, total_bytes_, 0, handles_[p], 0);
    }
    if (r == CUDA_SUCCESS) r = api->MemSetAccess(va, total_bytes_, &access, 1);
    if (r != CUDA_SUCCESS) {
      ok = false;
      err = "mapping peer memory failed (no P2P access?): " + DriverErrorString(api, r);
    }
  }
  for (auto& kv : peer_fds) close(kv.second);
  if (my_fd >= 0) close(my_fd);
  if (ok) {
    ok = cudaMemset(reinterpret_cast<void*>(vas_[rank]), 0, total_bytes_) == cudaSuccess &&
         cudaDeviceSynchronize() == cudaSuccess;
    if (!ok) err = "cudaMemset of the symmetric buffer failed";
  }
  if (!Agree(comm, ok)) {
    if (mc_fd >= 0) close(mc_fd);
    Destroy();
    return Status::PreconditionError("symmetric memory unavailable: " +
                                     (err.empty() ? "a peer reported failure" : err));
  }

  // 4. multicast: add devices, bind, map
  bool mc_ok = use_mc && (rank == 0 ? mc_fd >= 0 : mc_tag == 2);
  if (use_mc) {
    if (mc_ok && rank != 0) {
      r = api->MemImportFromShareableHandle(
          &mc_handle, reinterpret_cast<void*>(static_cast<intptr_t>(mc_fd)),
          CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      mc_ok = r == CUDA_SUCCESS;
    }
    if (mc_fd >= 0) close(mc_fd);
    if (mc_ok) {
      mc_handle_ = mc_handle;
      r = api->MulticastAddDevice(mc_handle, cudev);
      mc_ok = r == CUDA_SUCCESS;
    }
    mc_ok = Agree(comm, mc_ok);  // every device added before anyone binds
    if (mc_ok) {
      r = api->MulticastBindMem(mc_handle, 0, handles_[rank], 0, total_bytes_, 0);
      mc_ok = r == CUDA_SUCCESS;
      mc_bound_ = mc_ok;
    }
    if (mc_ok) {
      CUdeviceptr va = 0;
      r = api->MemAddressReserve(&va, total_bytes_, gran, 0, 0);
      if (r == CUDA_SUCCESS) {
        mc_va_ = va;
        r = api->MemMap(va, total_bytes_, 0, mc_handle, 0);
      }
      if (r == CUDA_SUCCESS) r = api->MemSetAccess(va, total_bytes_, &access, 1);
      mc_ok = r == CUDA_SUCCESS;
    }
    if (!mc_ok && r != CUDA_SUCCESS)
      HVD_LOG(WARNING) << "NVLink multicast setup failed: "
                       << DriverErrorString(api, r);
    mc_ok = Agree(comm, mc_ok);
  }

  info_.rank = rank;
  info_.world = world;
  info_.device = device;
  info_.data_bytes = data_rounded;
  info_.signal_bytes = signal_bytes;
  info_.multicast = mc_ok;
  info_.local = reinterpret_cast<void*>(vas_[rank]);
  for (int p = 0; p < world; ++p) {
    info_.peers[p] = reinterpret_cast<void*>(vas_[p]);
    info_.flags[p] = reinterpret_cast<uint32_t*>(vas_[p] + data_rounded);
  }
  if (mc_ok) {
    info_.mc = reinterpret_cast<void*>(mc_va_);
    info_.mc_flags = reinterpret_cast<uint32_t*>(mc_va_ + data_rounded);
  }
  comm.Barrier();
  return Status::OK();
}

void SymmArena::Destroy() {
  const DriverApi* api = GetDriverApi(nullptr);
  if (api != nullptr) {
    if (mc_va_) {
      api->MemUnmap(mc_va_, total_bytes_);
      api->MemAddressFree(mc_va_, total_bytes_);
    }
    if (mc_handle_) {
      if (mc_bound_) {
        CUdevice dev = 0;
        if (api->DeviceGet(&dev, info_.device) == CUDA_SUCCESS)
          api->MulticastUnbind(mc_handle_, dev, 0, total_bytes_);
      }
      api->MemRelease(mc_handle_);
    }
    for (size_t p = 0; p < vas_.size(); ++p) {
      if (vas_[p]) {
        api->MemUnmap(vas_[p], total_bytes_);
        api->MemAddressFree(vas_[p], total_bytes_);
      }
    }
    for (auto h : handles_)
      if (h) api->MemRelease(h);
  }
  handles_.clear();
  vas_.clear();
  mc_handle_ = 0;
  mc_va_ = 0;
  mc_bound_ = false;
  total_bytes_ = 0;
  info_ = SymmArenaInfo();
}

}  // namespace hvd
