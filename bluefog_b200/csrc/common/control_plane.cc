#include "control_plane.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <thread>

#include "logging.h"

namespace bfb {
namespace {

double NowS() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

void SetNoDelay(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  int buf = 4 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

void SetNonBlocking(int fd, bool on) {
  int flags = fcntl(fd, F_GETFL, 0);
  if (on)
    fcntl(fd, F_SETFL, flags | O_NONBLOCK);
  else
    fcntl(fd, F_SETFL, flags & ~O_NONBLOCK);
}

Status WriteAll(int fd, const void* data, size_t n, double deadline) {
  const char* p = static_cast<const char*>(data);
  while (n > 0) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w > 0) {
      p += w;
      n -= static_cast<size_t>(w);
      continue;
    }
    if (w < 0 && (errno == EINTR)) continue;
    if (w < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) {
      if (deadline > 0 && NowS() > deadline) return Status::Aborted("control plane: send timed out");
      struct pollfd pfd = {fd, POLLOUT, 0};
      poll(&pfd, 1, 100);
      continue;
    }
    return Status::Aborted(std::string("control plane: send failed: ") + std::strerror(errno));
  }
  return Status::OK();
}

Status ReadAll(int fd, void* data, size_t n, double deadline) {
  char* p = static_cast<char*>(data);
  while (n > 0) {
    struct pollfd pfd = {fd, POLLIN, 0};
    int pr = poll(&pfd, 1, 100);
    if (pr == 0) {
      if (deadline > 0 && NowS() > deadline) return Status::Aborted("control plane: receive timed out");
      continue;
    }
    if (pr < 0) {
      if (errno == EINTR) continue;
      return Status::Aborted(std::string("control plane: poll failed: ") + std::strerror(errno));
    }
    ssize_t r = ::recv(fd, p, n, 0);
    if (r > 0) {
      p += r;
      n -= static_cast<size_t>(r);
      continue;
    }
    if (r == 0) return Status::Aborted("control plane: peer closed the connection");
    if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
    return Status::Aborted(std::string("control plane: recv failed: ") + std::strerror(errno));
  }
  return Status::OK();
}

}  // namespace

ControlPlane::~ControlPlane() { Close(); }

void ControlPlane::Close() {
  for (auto& chan : fds_)
    for (int& fd : chan)
      if (fd >= 0) {
        ::shutdown(fd, SHUT_RDWR);
        ::close(fd);
        fd = -1;
      }
  fds_.clear();
  if (listen_fd_ >= 0) {
    ::close(listen_fd_);
    listen_fd_ = -1;
  }
  connected_ = false;
}

Status ControlPlane::Listen(const std::string& bind_addr, int* port) {
  listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
  if (listen_fd_ < 0) return Status::UnknownError("control plane: socket() failed");
  int one = 1;
  setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  struct sockaddr_in addr;
  std::memset(&addr, 0, sizeof(addr));
  addr.sin_family = AF_INET;
  addr.sin_port = 0;
  if (bind_addr.empty() || inet_pton(AF_INET, bind_addr.c_str(), &addr.sin_addr) != 1)
    addr.sin_addr.s_addr = htonl(INADDR_ANY);
  if (::bind(listen_fd_, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) != 0)
    return Status::UnknownError(std::string("control plane: bind failed: ") + std::strerror(errno));
  if (::listen(listen_fd_, 1024) != 0)
    return Status::UnknownError(std::string("control plane: listen failed: ") + std::strerror(errno));
  socklen_t len = sizeof(addr);
  getsockname(listen_fd_, reinterpret_cast<struct sockaddr*>(&addr), &len);
  *port = ntohs(addr.sin_port);
  return Status::OK();
}

Status ControlPlane::Connect(int rank, int size, const std::vector<std::string>& endpoints,
                             double timeout_s) {
  rank_ = rank;
  size_ = size;
  fds_.assign(kNumChannels, std::vector<int>(size, -1));
  if (static_cast<int>(endpoints.size()) != size)
    return Status::InvalidArgument("control plane: endpoint list does not match the world size");
  const double deadline = NowS() + timeout_s;

  // Active side: connect to every lower rank, once per channel, and announce (rank, channel).
  for (int peer = 0; peer < rank; ++peer) {
    const std::string& ep = endpoints[peer];
    auto colon = ep.rfind(':');
    if (colon == std::string::npos) return Status::InvalidArgument("control plane: bad endpoint " + ep);
    std::string host = ep.substr(0, colon);
    std::string port = ep.substr(colon + 1);
    struct addrinfo hints, *res = nullptr;
    std::memset(&hints, 0, sizeof(hints));
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    if (getaddrinfo(host.c_str(), port.c_str(), &hints, &res) != 0 || res == nullptr)
      return Status::UnknownError("control plane: cannot resolve " + ep);
    for (int ch = 0; ch < kNumChannels; ++ch) {
      int fd = -1;
      for (;;) {
        fd = ::socket(AF_INET, SOCK_STREAM, 0);
        if (::connect(fd, res->ai_addr, res->ai_addrlen) == 0) break;
        ::close(fd);
        fd = -1;
        if (NowS() > deadline) {
          freeaddrinfo(res);
          return Status::Aborted("control plane: timed out connecting to rank " + std::to_string(peer));
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(20));
      }
      SetNoDelay(fd);
      int32_t hello[2] = {rank, ch};
      Status s = WriteAll(fd, hello, sizeof(hello), deadline);
      if (!s.ok()) {
        freeaddrinfo(res);
        return s;
      }
      fds_[ch][peer] = fd;
    }
    freeaddrinfo(res);
  }
  // Passive side: accept from every higher rank.
  int expected = (size - 1 - rank) * kNumChannels;
  while (expected > 0) {
    struct pollfd pfd = {listen_fd_, POLLIN, 0};
    int pr = poll(&pfd, 1, 100);
    if (pr <= 0) {
      if (NowS() > deadline) return Status::Aborted("control plane: timed out waiting for peers to connect");
      continue;
    }
    int fd = ::accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) continue;
    SetNoDelay(fd);
    int32_t hello[2];
    Status s = ReadAll(fd, hello, sizeof(hello), deadline);
    if (!s.ok()) return s;
    if (hello[0] <= rank || hello[0] >= size || hello[1] < 0 || hello[1] >= kNumChannels ||
        fds_[hello[1]][hello[0]] != -1) {
      ::close(fd);
      return Status::UnknownError("control plane: unexpected handshake");
    }
    fds_[hello[1]][hello[0]] = fd;
    --expected;
  }
  for (auto& chan : fds_)
    for (int fd : chan)
      if (fd >= 0) SetNonBlocking(fd, true);
  connected_ = true;
  return Status::OK();
}

Status ControlPlane::SendMsg(int channel, int peer, const std::string& bytes) {
  int fd = fds_[channel][peer];
  if (fd < 0) return Status::Aborted("control plane: no connection to rank " + std::to_string(peer));
  const double deadline = NowS() + default_timeout_s;
  uint64_t n = bytes.size();
  Status s = WriteAll(fd, &n, sizeof(n), deadline);
  if (!s.ok()) return s;
  return WriteAll(fd, bytes.data(), bytes.size(), deadline);
}

Status ControlPlane::RecvMsg(int channel, int peer, std::string* bytes, double timeout_s) {
  int fd = fds_[channel][peer];
  if (fd < 0) return Status::Aborted("control plane: no connection to rank " + std::to_string(peer));
  const double deadline = NowS() + (timeout_s > 0 ? timeout_s : default_timeout_s);
  uint64_t n = 0;
  Status s = ReadAll(fd, &n, sizeof(n), deadline);
  if (!s.ok()) return s;
  bytes->resize(n);
  if (n == 0) return Status::OK();
  return ReadAll(fd, &(*bytes)[0], n, deadline);
}

Status ControlPlane::Exchange(int channel, const std::vector<SendSpec>& sends,
                              const std::vector<RecvSpec>& recvs, double timeout_s) {
  struct Prog {
    int fd;
    char* p;
    size_t left;
    bool is_send;
    int peer;
  };
  std::vector<Prog> prog;
  for (const auto& s : sends) {
    if (s.peer == rank_) return Status::InvalidArgument("control plane: send to self");
    if (s.nbytes) prog.push_back({fds_[channel][s.peer], const_cast<char*>(static_cast<const char*>(s.data)), s.nbytes, true, s.peer});
  }
  for (const auto& r : recvs) {
    if (r.peer == rank_) return Status::InvalidArgument("control plane: receive from self");
    if (r.nbytes) prog.push_back({fds_[channel][r.peer], static_cast<char*>(r.data), r.nbytes, false, r.peer});
  }
  const double deadline = NowS() + (timeout_s > 0 ? timeout_s : default_timeout_s);
  size_t remaining = prog.size();
  std::vector<struct pollfd> pfds;
  std::vector<size_t> index;
  while (remaining > 0) {
    pfds.clear();
    index.clear();
    // Per socket only the first unfinished send and the first unfinished receive may progress,
    // so that frames on one stream keep their posting order.
    for (size_t i = 0; i < prog.size(); ++i) {
      if (prog[i].left == 0) continue;
      bool blocked = false;
      for (size_t j = 0; j < i; ++j)
        if (prog[j].left && prog[j].fd == prog[i].fd && prog[j].is_send == prog[i].is_send) blocked = true;
      if (blocked) continue;
      if (prog[i].fd < 0) return Status::Aborted("control plane: no connection to rank " + std::to_string(prog[i].peer));
      pfds.push_back({prog[i].fd, static_cast<short>(prog[i].is_send ? POLLOUT : POLLIN), 0});
      index.push_back(i);
    }
    int pr = poll(pfds.data(), pfds.size(), 100);
    if (pr < 0 && errno != EINTR) return Status::Aborted("control plane: poll failed");
    if (pr == 0 && NowS() > deadline) return Status::Aborted("control plane: exchange timed out");
    for (size_t k = 0; k < pfds.size(); ++k) {
      if (!pfds[k].revents) continue;
      Prog& g = prog[index[k]];
      ssize_t n = g.is_send ? ::send(g.fd, g.p, g.left, MSG_NOSIGNAL) : ::recv(g.fd, g.p, g.left, 0);
      if (n > 0) {
        g.p += n;
        g.left -= static_cast<size_t>(n);
        if (g.left == 0) --remaining;
      } else if (n == 0 && !g.is_send) {
        return Status::Aborted("control plane: rank " + std::to_string(g.peer) + " closed the connection");
      } else if (n < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) {
        return Status::Aborted("control plane: IO with rank " + std::to_string(g.peer) + " failed: " + std::strerror(errno));
      }
    }
  }
  return Status::OK();
}

Status ControlPlane::AllgatherBytes(int channel, const std::string& mine, std::vector<std::string>* all,
                                    double timeout_s) {
  all->assign(size_, std::string());
  (*all)[rank_] = mine;
  if (size_ == 1) return Status::OK();
  std::vector<uint64_t> sizes(size_, 0);
  uint64_t my_size = mine.size();
  sizes[rank_] = my_size;
  std::vector<SendSpec> sends;
  std::vector<RecvSpec> recvs;
  for (int p = 0; p < size_; ++p) {
    if (p == rank_) continue;
    sends.push_back({p, &my_size, sizeof(my_size)});
    recvs.push_back({p, &sizes[p], sizeof(uint64_t)});
  }
  Status s = Exchange(channel, sends, recvs, timeout_s);
  if (!s.ok()) return s;
  sends.clear();
  recvs.clear();
  for (int p = 0; p < size_; ++p) {
    if (p == rank_) continue;
    (*all)[p].resize(sizes[p]);
    sends.push_back({p, mine.data(), mine.size()});
    recvs.push_back({p, &(*all)[p][0], static_cast<size_t>(sizes[p])});
  }
  return Exchange(channel, sends, recvs, timeout_s);
}

Status ControlPlane::Barrier(int channel, double timeout_s) {
  std::vector<std::string> all;
  return AllgatherBytes(channel, std::string("b"), &all, timeout_s);
}

Status ControlPlane::BroadcastBytes(int channel, int root, std::string* bytes) {
  if (size_ == 1) return Status::OK();
  if (rank_ == root) {
    for (int p = 0; p < size_; ++p) {
      if (p == root) continue;
      Status s = SendMsg(channel, p, *bytes);
      if (!s.ok()) return s;
    }
    return Status::OK();
  }
  return RecvMsg(channel, root, bytes);
}

}  // namespace bfb
