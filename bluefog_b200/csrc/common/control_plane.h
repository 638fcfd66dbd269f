// TCP full-mesh transport between the ranks of one job.
//
// This is the host-side "MPI replacement": it carries the negotiation protocol, the
// exchange of CUDA IPC handles, barriers, and the CPU data path of every collective
// (role of bluefog/common/mpi_context.cc + the two-sided parts of mpi_controller.cc in
// the reference).  Every pair of ranks is joined by kNumChannels independent sockets so
// that the negotiation loop, the data path and the calling thread never interleave
// frames on one stream.  All blocking calls carry a deadline and report a peer that
// closed its socket as Status::Aborted, which is how a vanished rank is detected.
#pragma once
#include <cstdint>
#include <mutex>
#include <string>
#include <vector>

#include "status.h"

namespace bfb {

enum MeshChannel : int { kChanNegotiate = 0, kChanData = 1, kChanUser = 2, kNumChannels = 3 };

struct SendSpec {
  int peer;
  const void* data;
  size_t nbytes;
};
struct RecvSpec {
  int peer;
  void* data;
  size_t nbytes;
};

class ControlPlane {
 public:
  ControlPlane() = default;
  ~ControlPlane();
  ControlPlane(const ControlPlane&) = delete;

  // Step 1: open a listening socket on an ephemeral port of bind_addr; returns the port.
  Status Listen(const std::string& bind_addr, int* port);
  // Step 2: endpoints[i] = "host:port" of rank i (exchanged by the launcher-provided store).
  Status Connect(int rank, int size, const std::vector<std::string>& endpoints, double timeout_s);
  void Close();
  bool connected() const { return connected_; }
  int rank() const { return rank_; }
  int size() const { return size_; }

  // Raw socket of (channel, peer) for poll()-based event loops.
  int fd(int channel, int peer) const { return fds_[channel][peer]; }

  // Blocking framed messages: 8-byte little-endian length + payload.
  Status SendMsg(int channel, int peer, const std::string& bytes);
  Status RecvMsg(int channel, int peer, std::string* bytes, double timeout_s = -1);

  // Progresses all sends and receives together (poll + non-blocking IO): safe for any
  // communication pattern, including a pair that sends large buffers to each other.
  Status Exchange(int channel, const std::vector<SendSpec>& sends, const std::vector<RecvSpec>& recvs,
                  double timeout_s = -1);

  // Collectives on the user/data channel built from Exchange.
  Status AllgatherBytes(int channel, const std::string& mine, std::vector<std::string>* all, double timeout_s = -1);
  Status Barrier(int channel, double timeout_s = -1);
  Status BroadcastBytes(int channel, int root, std::string* bytes);

  double default_timeout_s = 300.0;

 private:
  int listen_fd_ = -1;
  int rank_ = 0, size_ = 1;
  bool connected_ = false;
  std::vector<std::vector<int>> fds_;  // [channel][peer]
  std::mutex user_mu_;
};

}  // namespace bfb
