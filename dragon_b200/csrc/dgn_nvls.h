// NVSwitch multicast ("NVLS") staging buffers: allocation with the CUDA
// virtual-memory API, one multicast object per communicator, every rank's
// buffer bound to it and mapped twice (own mapping and multicast mapping).
// Driver entry points are resolved at run time through
// cudaGetDriverEntryPoint, so the library does not link libcuda.
#pragma once

#include <stddef.h>

#include <string>

namespace dgn {

struct NvlsBuffer;  // one rank's share

// 1 if `device` can take part in a multicast object.
bool nvls_device_supported(int device);

// Ranks that all live in the calling process (one per entry of `devices`):
// creates the multicast object, binds and maps every rank's buffer.
// Returns 0 and fills out[0..n) on success.
int nvls_setup_inprocess(int n, const int* devices, size_t bytes, NvlsBuffer** out, std::string* err);

// One process per rank.  Rank 0 creates the multicast object and a listening
// abstract unix socket (name returned in `sockname`, at most 63 characters)
// before handles are exchanged; afterwards rank 0 calls nvls_root_finish and
// the others nvls_peer_join.  The file descriptor of the multicast object
// travels over the socket; the two sides also agree, in two rounds, that
// every rank added its device and bound its buffer.  All of them succeed or
// all of them fail.
int nvls_root_prepare(int device, int nranks, size_t bytes, NvlsBuffer** out, char* sockname, std::string* err);
int nvls_root_finish(NvlsBuffer* buf, int timeout_ms, std::string* err);
int nvls_peer_join(int device, int nranks, size_t bytes, const char* sockname, int timeout_ms, NvlsBuffer** out,
                   std::string* err);

void nvls_pointers(const NvlsBuffer* buf, char** unicast, char** multicast);
void nvls_destroy(NvlsBuffer* buf);

}  // namespace dgn
