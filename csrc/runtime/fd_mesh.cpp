// File-descriptor exchange between the ranks of one host: each rank binds one AF_UNIX datagram
// socket; a descriptor travels as SCM_RIGHTS ancillary data of a small message that names the
// sender and a tag. Datagram sockets need no connect/accept ordering, so the reference's
// "higher rank sends first" rule (iris/host/distributed/fd_passing.py:81-140, symmetric_heap.py:
// 263-269) has no counterpart here: every rank sends to all peers, then receives world-1 messages.
// Used for CUDA VMM POSIX handles, multicast handles and the memfd of the CPU backend.
#include <errno.h>
#include <poll.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <string>

namespace {
struct Mesh {
  int sock = -1;
  std::string path;
};
struct Msg {
  int32_t src;
  int32_t tag;
  uint64_t payload;
};
}  // namespace

extern "C" {

void* iris_fdmesh_create(const char* path, char* err, int errlen) {
  Mesh* m = new Mesh();
  m->path = path;
  m->sock = socket(AF_UNIX, SOCK_DGRAM, 0);
  if (m->sock < 0) {
    snprintf(err, errlen, "socket: %s", strerror(errno));
    delete m;
    return nullptr;
  }
  sockaddr_un addr;
  memset(&addr, 0, sizeof(addr));
  addr.sun_family = AF_UNIX;
  if (m->path.size() >= sizeof(addr.sun_path)) {
    snprintf(err, errlen, "socket path too long");
    close(m->sock);
    delete m;
    return nullptr;
  }
  strcpy(addr.sun_path, m->path.c_str());
  unlink(m->path.c_str());
  if (bind(m->sock, (sockaddr*)&addr, sizeof(addr)) != 0) {
    snprintf(err, errlen, "bind(%s): %s", m->path.c_str(), strerror(errno));
    close(m->sock);
    delete m;
    return nullptr;
  }
  return m;
}

// Send `fd` (or no descriptor when fd < 0) with (src, tag, payload) to the socket at `peer_path`.
int iris_fdmesh_send(void* mp, const char* peer_path, int fd, int src, int tag, uint64_t payload, char* err, int errlen) {
  Mesh* m = (Mesh*)mp;
  sockaddr_un addr;
  memset(&addr, 0, sizeof(addr));
  addr.sun_family = AF_UNIX;
  strncpy(addr.sun_path, peer_path, sizeof(addr.sun_path) - 1);
  Msg msg{src, tag, payload};
  iovec iov{&msg, sizeof(msg)};
  msghdr mh;
  memset(&mh, 0, sizeof(mh));
  mh.msg_name = &addr;
  mh.msg_namelen = sizeof(addr);
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  if (fd >= 0) {
    memset(ctrl, 0, sizeof(ctrl));
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&mh);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  // the peer may not have bound yet: retry for up to ~10 s (the reference's connect deadline)
  for (int attempt = 0; attempt < 1000; ++attempt) {
    if (sendmsg(m->sock, &mh, 0) >= 0) return 0;
    if (errno != ENOENT && errno != ECONNREFUSED && errno != EAGAIN && errno != ENOBUFS) break;
    usleep(10000);
  }
  snprintf(err, errlen, "sendmsg(%s): %s", peer_path, strerror(errno));
  return -1;
}

// Receive one message. Returns 0 and fills the outputs (fd = -1 when none came), -2 on timeout.
int iris_fdmesh_recv(void* mp, int timeout_ms, int* fd, int* src, int* tag, uint64_t* payload, char* err, int errlen) {
  Mesh* m = (Mesh*)mp;
  pollfd pfd{m->sock, POLLIN, 0};
  int pr = poll(&pfd, 1, timeout_ms);
  if (pr == 0) {
    snprintf(err, errlen, "timed out after %d ms waiting for a peer's descriptor", timeout_ms);
    return -2;
  }
  if (pr < 0) {
    snprintf(err, errlen, "poll: %s", strerror(errno));
    return -1;
  }
  Msg msg;
  iovec iov{&msg, sizeof(msg)};
  msghdr mh;
  memset(&mh, 0, sizeof(mh));
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  mh.msg_control = ctrl;
  mh.msg_controllen = sizeof(ctrl);
  ssize_t n = recvmsg(m->sock, &mh, 0);
  if (n != (ssize_t)sizeof(msg)) {
    snprintf(err, errlen, "recvmsg: short or failed read (%zd): %s", n, strerror(errno));
    return -1;
  }
  *fd = -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&mh); c; c = CMSG_NXTHDR(&mh, c))
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(fd, CMSG_DATA(c), sizeof(int));
  *src = msg.src;
  *tag = msg.tag;
  *payload = msg.payload;
  return 0;
}

void iris_fdmesh_destroy(void* mp) {
  Mesh* m = (Mesh*)mp;
  if (m->sock >= 0) close(m->sock);
  unlink(m->path.c_str());
  delete m;
}

void iris_close_fd(int fd) {
  if (fd >= 0) close(fd);
}

}  // extern "C"
