// NVSwitch multicast staging buffers (see dgn_nvls.h).
#include "dgn_nvls.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <poll.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <memory>
#include <vector>

namespace dgn {

namespace {

// ---- driver entry points ---------------------------------------------------

struct Driver {
  bool ok = false;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                               unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                         unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
};

template <typename F>
bool resolve(const char* name, F* fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    cudaGetLastError();
    return false;
  }
  *fn = reinterpret_cast<F>(p);
  return true;
}

const Driver& driver() {
  static Driver d = [] {
    Driver x;
    x.ok = resolve("cuDeviceGet", &x.DeviceGet) && resolve("cuDeviceGetAttribute", &x.DeviceGetAttribute) &&
           resolve("cuMulticastCreate", &x.MulticastCreate) && resolve("cuMulticastAddDevice", &x.MulticastAddDevice) &&
           resolve("cuMulticastBindMem", &x.MulticastBindMem) && resolve("cuMulticastUnbind", &x.MulticastUnbind) &&
           resolve("cuMulticastGetGranularity", &x.MulticastGetGranularity) && resolve("cuMemCreate", &x.MemCreate) &&
           resolve("cuMemRelease", &x.MemRelease) && resolve("cuMemAddressReserve", &x.MemAddressReserve) &&
           resolve("cuMemAddressFree", &x.MemAddressFree) && resolve("cuMemMap", &x.MemMap) &&
           resolve("cuMemUnmap", &x.MemUnmap) && resolve("cuMemSetAccess", &x.MemSetAccess) &&
           resolve("cuMemExportToShareableHandle", &x.MemExportToShareableHandle) &&
           resolve("cuMemImportFromShareableHandle", &x.MemImportFromShareableHandle) &&
           resolve("cuMemGetAllocationGranularity", &x.MemGetAllocationGranularity);
    return x;
  }();
  return d;
}

int fail(std::string* err, const char* what, CUresult r) {
  if (err) {
    char buf[160];
    snprintf(buf, sizeof(buf), "%s failed (CUresult %d)", what, (int)r);
    *err = buf;
  }
  return 1;
}
int fail(std::string* err, const char* what) {
  if (err) *err = what;
  return 1;
}

#define NV_CHECK(call, what)                      \
  do {                                            \
    CUresult r__ = (call);                        \
    if (r__ != CUDA_SUCCESS) return fail(err, what, r__); \
  } while (0)

double now_s() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

CUmulticastObjectProp mc_prop(int nranks, size_t bytes) {
  CUmulticastObjectProp p;
  memset(&p, 0, sizeof(p));
  p.numDevices = (unsigned)nranks;
  p.size = bytes;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

CUmemAllocationProp mem_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

// Size rounded to what both the multicast object and the allocation accept.
int padded_size(int nranks, int device, size_t bytes, size_t* out, std::string* err) {
  const Driver& d = driver();
  size_t g_mc = 0, g_mem = 0;
  CUmulticastObjectProp mp = mc_prop(nranks, bytes);
  NV_CHECK(d.MulticastGetGranularity(&g_mc, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
  CUmemAllocationProp ap = mem_prop(device);
  NV_CHECK(d.MemGetAllocationGranularity(&g_mem, &ap, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
           "cuMemGetAllocationGranularity");
  size_t g = g_mc > g_mem ? g_mc : g_mem;
  if (g == 0) g = 2u << 20;
  *out = (bytes + g - 1) / g * g;
  return 0;
}

std::atomic<int> g_socket_seq{0};

}  // namespace

// The multicast object is released when the last buffer that uses the
// handle is gone: ranks of one process share one handle, and a rank must
// unbind before the object goes away.
struct McRef {
  CUmemGenericAllocationHandle handle;
  explicit McRef(CUmemGenericAllocationHandle h) : handle(h) {}
  ~McRef();
};

struct NvlsBuffer {
  std::shared_ptr<McRef> mc_ref;
  int device = 0, nranks = 0;
  size_t bytes = 0;
  CUmemGenericAllocationHandle mem = 0, mc = 0;
  bool has_mem = false, bound = false;
  CUdeviceptr uva = 0, mva = 0;
  bool uva_mapped = false, mva_mapped = false;
  int listen_fd = -1;
  std::vector<int> peers;  // root: one connected socket per other rank
};

namespace {

// With `b->device` current: add the device to the multicast object.
int add_device(NvlsBuffer* b, std::string* err) {
  const Driver& d = driver();
  CUdevice dev;
  NV_CHECK(d.DeviceGet(&dev, b->device), "cuDeviceGet");
  NV_CHECK(d.MulticastAddDevice(b->mc, dev), "cuMulticastAddDevice");
  return 0;
}

// With `b->device` current and every device added: allocate, bind, map twice.
int bind_and_map(NvlsBuffer* b, std::string* err) {
  const Driver& d = driver();
  CUmemAllocationProp ap = mem_prop(b->device);
  NV_CHECK(d.MemCreate(&b->mem, b->bytes, &ap, 0), "cuMemCreate");
  b->has_mem = true;
  NV_CHECK(d.MulticastBindMem(b->mc, 0, b->mem, 0, b->bytes, 0), "cuMulticastBindMem");
  b->bound = true;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = b->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  NV_CHECK(d.MemAddressReserve(&b->uva, b->bytes, 0, 0, 0), "cuMemAddressReserve");
  NV_CHECK(d.MemMap(b->uva, b->bytes, 0, b->mem, 0), "cuMemMap");
  b->uva_mapped = true;
  NV_CHECK(d.MemSetAccess(b->uva, b->bytes, &acc, 1), "cuMemSetAccess");
  NV_CHECK(d.MemAddressReserve(&b->mva, b->bytes, 0, 0, 0), "cuMemAddressReserve (multicast)");
  NV_CHECK(d.MemMap(b->mva, b->bytes, 0, b->mc, 0), "cuMemMap (multicast)");
  b->mva_mapped = true;
  NV_CHECK(d.MemSetAccess(b->mva, b->bytes, &acc, 1), "cuMemSetAccess (multicast)");
  if (cudaMemset(reinterpret_cast<void*>(b->uva), 0, b->bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    return fail(err, "clearing the multicast staging buffer failed");
  }
  return 0;
}

// ---- socket helpers --------------------------------------------------------------

bool wait_fd(int fd, short events, double deadline) {
  for (;;) {
    double left = deadline - now_s();
    if (left <= 0) return false;
    struct pollfd p = {fd, events, 0};
    int rc = poll(&p, 1, (int)(left * 1000) + 1);
    if (rc > 0) return true;
    if (rc < 0 && errno != EINTR) return false;
  }
}

bool send_all(int fd, const void* data, size_t n) {
  const char* p = static_cast<const char*>(data);
  while (n > 0) {
    ssize_t k = send(fd, p, n, MSG_NOSIGNAL);
    if (k <= 0) {
      if (k < 0 && errno == EINTR) continue;
      return false;
    }
    p += k;
    n -= (size_t)k;
  }
  return true;
}

bool recv_all(int fd, void* data, size_t n, double deadline) {
  char* p = static_cast<char*>(data);
  while (n > 0) {
    if (!wait_fd(fd, POLLIN, deadline)) return false;
    ssize_t k = recv(fd, p, n, 0);
    if (k <= 0) {
      if (k < 0 && errno == EINTR) continue;
      return false;
    }
    p += k;
    n -= (size_t)k;
  }
  return true;
}

bool send_fd(int sock, int fd) {
  char byte = 'F';
  struct iovec iov = {&byte, 1};
  char ctl[CMSG_SPACE(sizeof(int))];
  memset(ctl, 0, sizeof(ctl));
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctl;
  msg.msg_controllen = sizeof(ctl);
  struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return sendmsg(sock, &msg, MSG_NOSIGNAL) == 1;
}

int recv_fd(int sock, double deadline) {
  if (!wait_fd(sock, POLLIN, deadline)) return -1;
  char byte = 0;
  struct iovec iov = {&byte, 1};
  char ctl[CMSG_SPACE(sizeof(int))];
  memset(ctl, 0, sizeof(ctl));
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctl;
  msg.msg_controllen = sizeof(ctl);
  if (recvmsg(sock, &msg, 0) != 1) return -1;
  struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return -1;
  int fd = -1;
  memcpy(&fd, CMSG_DATA(c), sizeof(int));
  return fd;
}

socklen_t abstract_address(const char* name, struct sockaddr_un* addr) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  size_t n = strlen(name);
  if (n > sizeof(addr->sun_path) - 2) n = sizeof(addr->sun_path) - 2;
  memcpy(addr->sun_path + 1, name, n);  // leading NUL: abstract namespace, nothing on disk
  return (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + n);
}

}  // namespace

McRef::~McRef() { driver().MemRelease(handle); }

bool nvls_device_supported(int device) {
  const Driver& d = driver();
  if (!d.ok) return false;
  CUdevice dev;
  if (d.DeviceGet(&dev, device) != CUDA_SUCCESS) return false;
  int v = 0;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return false;
  return v != 0;
}

void nvls_pointers(const NvlsBuffer* b, char** unicast, char** multicast) {
  *unicast = reinterpret_cast<char*>(b->uva);
  *multicast = reinterpret_cast<char*>(b->mva);
}

void nvls_destroy(NvlsBuffer* b) {
  if (!b) return;
  const Driver& d = driver();
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(b->device);
  cudaDeviceSynchronize();
  if (b->mva_mapped) d.MemUnmap(b->mva, b->bytes);
  if (b->mva) d.MemAddressFree(b->mva, b->bytes);
  if (b->bound) {
    CUdevice dev;
    if (d.DeviceGet(&dev, b->device) == CUDA_SUCCESS) d.MulticastUnbind(b->mc, dev, 0, b->bytes);
  }
  if (b->uva_mapped) d.MemUnmap(b->uva, b->bytes);
  if (b->uva) d.MemAddressFree(b->uva, b->bytes);
  if (b->has_mem) d.MemRelease(b->mem);
  b->mc_ref.reset();
  for (int fd : b->peers) close(fd);
  if (b->listen_fd >= 0) close(b->listen_fd);
  cudaSetDevice(prev);
  delete b;
}

int nvls_setup_inprocess(int n, const int* devices, size_t bytes, NvlsBuffer** out, std::string* err) {
  const Driver& d = driver();
  if (!d.ok) return fail(err, "multicast driver entry points are not available");
  for (int r = 0; r < n; ++r) {
    out[r] = nullptr;
    if (!nvls_device_supported(devices[r])) return fail(err, "a device does not support multicast");
    for (int q = 0; q < r; ++q)
      if (devices[q] == devices[r]) return fail(err, "two ranks share a device");
  }
  int prev = 0;
  cudaGetDevice(&prev);
  size_t padded = 0;
  cudaSetDevice(devices[0]);
  if (padded_size(n, devices[0], bytes, &padded, err)) { cudaSetDevice(prev); return 1; }
  CUmemGenericAllocationHandle mc = 0;
  CUmulticastObjectProp mp = mc_prop(n, padded);
  CUresult cr = d.MulticastCreate(&mc, &mp);
  if (cr != CUDA_SUCCESS) { cudaSetDevice(prev); return fail(err, "cuMulticastCreate", cr); }
  std::shared_ptr<McRef> ref = std::make_shared<McRef>(mc);
  int rc = 0;
  std::vector<NvlsBuffer*> made;
  for (int r = 0; r < n && !rc; ++r) {
    NvlsBuffer* b = new NvlsBuffer();
    b->device = devices[r];
    b->nranks = n;
    b->bytes = padded;
    b->mc = mc;
    b->mc_ref = ref;
    made.push_back(b);
    cudaSetDevice(devices[r]);
    rc = add_device(b, err);
  }
  for (int r = 0; r < n && !rc; ++r) {
    cudaSetDevice(devices[r]);
    rc = bind_and_map(made[r], err);
  }
  cudaSetDevice(prev);
  if (rc) {
    for (size_t i = made.size(); i-- > 0;) nvls_destroy(made[i]);
    return 1;
  }
  for (int r = 0; r < n; ++r) out[r] = made[r];
  return 0;
}

int nvls_root_prepare(int device, int nranks, size_t bytes, NvlsBuffer** out, char* sockname, std::string* err) {
  *out = nullptr;
  const Driver& d = driver();
  if (!d.ok) return fail(err, "multicast driver entry points are not available");
  if (!nvls_device_supported(device)) return fail(err, "device does not support multicast");
  NvlsBuffer* b = new NvlsBuffer();
  b->device = device;
  b->nranks = nranks;
  if (padded_size(nranks, device, bytes, &b->bytes, err)) { delete b; return 1; }
  CUmulticastObjectProp mp = mc_prop(nranks, b->bytes);
  CUresult cr = d.MulticastCreate(&b->mc, &mp);
  if (cr != CUDA_SUCCESS) { delete b; return fail(err, "cuMulticastCreate", cr); }
  b->mc_ref = std::make_shared<McRef>(b->mc);
  snprintf(sockname, 64, "dgn-nvls-%d-%d", (int)getpid(), g_socket_seq.fetch_add(1));
  b->listen_fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  struct sockaddr_un addr;
  socklen_t len = abstract_address(sockname, &addr);
  if (b->listen_fd < 0 || bind(b->listen_fd, (struct sockaddr*)&addr, len) != 0 || listen(b->listen_fd, 16) != 0) {
    nvls_destroy(b);
    return fail(err, "cannot listen on the multicast rendezvous socket");
  }
  *out = b;
  return 0;
}

int nvls_root_finish(NvlsBuffer* b, int timeout_ms, std::string* err) {
  const Driver& d = driver();
  const double deadline = now_s() + 1e-3 * timeout_ms;
  int fd = -1;
  NV_CHECK(d.MemExportToShareableHandle(&fd, b->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
           "cuMemExportToShareableHandle");
  bool ok = true;
  for (int i = 0; i < b->nranks - 1 && ok; ++i) {
    if (!wait_fd(b->listen_fd, POLLIN, deadline)) { ok = false; break; }
    int s = accept(b->listen_fd, nullptr, nullptr);
    if (s < 0) { ok = false; break; }
    b->peers.push_back(s);
    ok = send_fd(s, fd);
  }
  close(fd);
  if (!ok) return fail(err, "a rank did not join the multicast rendezvous in time");
  // First exchange: every device added.  Second exchange: every buffer bound and mapped.
  for (int round = 0; round < 2; ++round) {
    char mine = (round == 0 ? add_device(b, err) : bind_and_map(b, err)) == 0 ? '1' : '0';
    char all = mine;
    for (int s : b->peers) {
      char c = '0';
      if (!recv_all(s, &c, 1, deadline)) c = '0';
      if (c != '1') all = '0';
    }
    for (int s : b->peers) send_all(s, &all, 1);
    if (all != '1') return fail(err, round == 0 ? "a rank could not add its device to the multicast object"
                                                 : "a rank could not bind its buffer to the multicast object");
  }
  return 0;
}

int nvls_peer_join(int device, int nranks, size_t bytes, const char* sockname, int timeout_ms, NvlsBuffer** out,
                   std::string* err) {
  *out = nullptr;
  const Driver& d = driver();
  const double deadline = now_s() + 1e-3 * timeout_ms;
  int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (s < 0) return fail(err, "socket() failed");
  struct sockaddr_un addr;
  socklen_t len = abstract_address(sockname, &addr);
  while (connect(s, (struct sockaddr*)&addr, len) != 0) {
    if (now_s() > deadline) { close(s); return fail(err, "cannot reach the multicast rendezvous socket"); }
    usleep(2000);
  }
  NvlsBuffer* b = new NvlsBuffer();
  b->device = device;
  b->nranks = nranks;
  b->peers.push_back(s);
  // Every step reports to the root even after a local failure, so that all
  // ranks leave the two rounds together.
  bool usable = d.ok && nvls_device_supported(device) && padded_size(nranks, device, bytes, &b->bytes, err) == 0;
  int fd = recv_fd(s, deadline);
  if (fd < 0) { nvls_destroy(b); return fail(err, "did not receive the multicast handle"); }
  if (usable) {
    CUresult cr = d.MemImportFromShareableHandle(&b->mc, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    if (cr != CUDA_SUCCESS) { usable = false; fail(err, "cuMemImportFromShareableHandle", cr); }
    else b->mc_ref = std::make_shared<McRef>(b->mc);
  }
  close(fd);
  for (int round = 0; round < 2; ++round) {
    if (usable) usable = (round == 0 ? add_device(b, err) : bind_and_map(b, err)) == 0;
    char mine = usable ? '1' : '0', all = '0';
    if (!send_all(s, &mine, 1) || !recv_all(s, &all, 1, deadline) || all != '1') {
      std::string keep = err ? *err : std::string();
      nvls_destroy(b);
      if (err && keep.empty()) *err = "another rank could not set up multicast";
      else if (err) *err = keep;
      return 1;
    }
  }
  *out = b;
  return 0;
}

}  // namespace dgn
