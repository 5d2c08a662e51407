#include "bootstrap.h"

#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <chrono>
#include <random>
#include <stdexcept>
#include <thread>

namespace penny {

namespace {

[[noreturn]] void fail(const std::string& what) {
  throw std::runtime_error("penny bootstrap: " + what + " (" + strerror(errno) + ")");
}

long long now_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

// Abstract-namespace address: no file on disk, vanishes with the process.
socklen_t make_addr(const std::string& uid, int rank, sockaddr_un* addr) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  std::string name = "penny-" + uid + "-" + std::to_string(rank);
  if (name.size() + 1 > sizeof(addr->sun_path)) name.resize(sizeof(addr->sun_path) - 1);
  addr->sun_path[0] = '\0';
  memcpy(addr->sun_path + 1, name.data(), name.size());
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

void wait_io(int fd, short events, long long deadline, const char* what) {
  for (;;) {
    long long left = deadline - now_ms();
    if (left <= 0) {
      errno = ETIMEDOUT;
      fail(std::string("timed out in ") + what);
    }
    pollfd p{fd, events, 0};
    int rc = poll(&p, 1, (int)(left > 1000 ? 1000 : left));
    if (rc > 0) return;
    if (rc < 0 && errno != EINTR) fail(std::string("poll in ") + what);
  }
}

}  // namespace

std::string make_unique_id() {
  std::random_device rd;
  static const char* hex = "0123456789abcdef";
  std::string s(32, '0');
  for (int i = 0; i < 32; i += 8) {
    unsigned v = rd() ^ (unsigned)(now_ms() * 2654435761u) ^ (unsigned)getpid() * 40503u;
    for (int j = 0; j < 8; ++j) s[i + j] = hex[(v >> (4 * j)) & 15];
  }
  return s;
}

Bootstrap::Bootstrap(const std::string& uid, int rank, int world, int timeout_ms)
    : rank_(rank), world_(world), timeout_ms_(timeout_ms), conn_(world, -1) {
  if (world < 1 || rank < 0 || rank >= world) {
    errno = EINVAL;
    fail("bad rank/world");
  }
  const long long deadline = now_ms() + timeout_ms_;
  listen_fd_ = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (listen_fd_ < 0) fail("socket");
  sockaddr_un addr;
  socklen_t len = make_addr(uid, rank, &addr);
  if (bind(listen_fd_, (sockaddr*)&addr, len) != 0) fail("bind");
  if (listen(listen_fd_, world) != 0) fail("listen");

  // connect to every lower rank (it may not be listening yet: retry) ...
  for (int p = 0; p < rank; ++p) {
    sockaddr_un pa;
    socklen_t pl = make_addr(uid, p, &pa);
    for (;;) {
      int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
      if (fd < 0) fail("socket");
      if (connect(fd, (sockaddr*)&pa, pl) == 0) {
        conn_[p] = fd;
        break;
      }
      close(fd);
      if (now_ms() > deadline) {
        errno = ETIMEDOUT;
        fail("connect to rank " + std::to_string(p));
      }
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    int me = rank;
    send_bytes(p, &me, sizeof(me));
  }
  // ... and accept every higher one
  for (int k = rank + 1; k < world; ++k) {
    wait_io(listen_fd_, POLLIN, deadline, "accept");
    int fd = accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
    if (fd < 0) fail("accept");
    int who = -1;
    size_t got = 0;
    while (got < sizeof(who)) {
      wait_io(fd, POLLIN, deadline, "hello");
      ssize_t n = read(fd, (char*)&who + got, sizeof(who) - got);
      if (n <= 0) fail("hello read");
      got += (size_t)n;
    }
    if (who <= rank || who >= world || conn_[who] != -1) {
      errno = EPROTO;
      fail("unexpected peer");
    }
    conn_[who] = fd;
  }
}

Bootstrap::~Bootstrap() {
  for (int fd : conn_)
    if (fd >= 0) close(fd);
  if (listen_fd_ >= 0) close(listen_fd_);
}

void Bootstrap::send_bytes(int peer, const void* p, size_t bytes) {
  const long long deadline = now_ms() + timeout_ms_;
  const char* c = (const char*)p;
  while (bytes > 0) {
    wait_io(conn_[peer], POLLOUT, deadline, "send");
    ssize_t n = send(conn_[peer], c, bytes, MSG_NOSIGNAL);
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      fail("send to rank " + std::to_string(peer));
    }
    c += n;
    bytes -= (size_t)n;
  }
}

void Bootstrap::recv_bytes(int peer, void* p, size_t bytes) {
  const long long deadline = now_ms() + timeout_ms_;
  char* c = (char*)p;
  while (bytes > 0) {
    wait_io(conn_[peer], POLLIN, deadline, "recv");
    ssize_t n = recv(conn_[peer], c, bytes, 0);
    if (n == 0) {
      errno = ECONNRESET;
      fail("rank " + std::to_string(peer) + " closed the connection");
    }
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      fail("recv from rank " + std::to_string(peer));
    }
    c += n;
    bytes -= (size_t)n;
  }
}

void Bootstrap::all_gather(const void* in, size_t bytes, void* out) {
  char* o = (char*)out;
  memcpy(o + (size_t)rank_ * bytes, in, bytes);
  // Socket buffers hold these small blobs, so send-all then receive-all cannot
  // deadlock for the sizes this is used with (handles, pointers, a few KB).
  for (int p = 0; p < world_; ++p)
    if (p != rank_) send_bytes(p, in, bytes);
  for (int p = 0; p < world_; ++p)
    if (p != rank_) recv_bytes(p, o + (size_t)p * bytes, bytes);
}

void Bootstrap::barrier() {
  char token = 1;
  std::vector<char> all(world_);
  all_gather(&token, 1, all.data());
}

void Bootstrap::send_fd(int peer, int fd) {
  const long long deadline = now_ms() + timeout_ms_;
  char payload = 'F';
  iovec iov{&payload, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* cm = CMSG_FIRSTHDR(&msg);
  cm->cmsg_level = SOL_SOCKET;
  cm->cmsg_type = SCM_RIGHTS;
  cm->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(cm), &fd, sizeof(int));
  for (;;) {
    wait_io(conn_[peer], POLLOUT, deadline, "send_fd");
    ssize_t n = sendmsg(conn_[peer], &msg, MSG_NOSIGNAL);
    if (n == 1) return;
    if (n < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    fail("sendmsg(fd) to rank " + std::to_string(peer));
  }
}

int Bootstrap::recv_fd(int peer) {
  const long long deadline = now_ms() + timeout_ms_;
  char payload = 0;
  iovec iov{&payload, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  for (;;) {
    wait_io(conn_[peer], POLLIN, deadline, "recv_fd");
    ssize_t n = recvmsg(conn_[peer], &msg, MSG_CMSG_CLOEXEC);
    if (n == 1) break;
    if (n < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    if (n == 0) errno = ECONNRESET;
    fail("recvmsg(fd) from rank " + std::to_string(peer));
  }
  cmsghdr* cm = CMSG_FIRSTHDR(&msg);
  if (!cm || cm->cmsg_level != SOL_SOCKET || cm->cmsg_type != SCM_RIGHTS || payload != 'F') {
    errno = EPROTO;
    fail("no descriptor in message from rank " + std::to_string(peer));
  }
  int fd = -1;
  memcpy(&fd, CMSG_DATA(cm), sizeof(int));
  return fd;
}

}  // namespace penny
