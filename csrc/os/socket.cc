#include "socket.h"

#include <arpa/inet.h>
#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <sys/un.h>
#include <unistd.h>

namespace mccl {

DEFINE_MCCL_PARAM(SocketBufKb, "SOCKET_BUF_KB", 4096);

static void tuneStream(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}

void sockSetBuffers(int fd, int bytes) {
  if (bytes <= 0) return;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &bytes, sizeof(bytes));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &bytes, sizeof(bytes));
}

void sockSetDeadline(int fd, int seconds) {
  struct timeval tv = {seconds, 0};
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
}

void sockSetKeepalive(int fd, int idleSec) {
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_KEEPALIVE, &one, sizeof(one));
  if (idleSec > 0) setsockopt(fd, IPPROTO_TCP, TCP_KEEPIDLE, &idleSec, sizeof(idleSec));
}

mcclResult_t sockListen(const char* ip, uint16_t port, int* fd, uint16_t* boundPort) {
  int s = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (s < 0) MCCLFAIL(mcclSystemError);
  int one = 1;
  setsockopt(s, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockSetBuffers(s, (int)(mcclParamSocketBufKb() * 1024));
  struct sockaddr_in a;
  memset(&a, 0, sizeof(a));
  a.sin_family = AF_INET;
  a.sin_port = htons(port);
  a.sin_addr.s_addr = htonl(INADDR_ANY);
  if (ip != nullptr && *ip && inet_pton(AF_INET, ip, &a.sin_addr) != 1) {
    close(s);
    MCCLFAIL(mcclInvalidArgument);
  }
  if (bind(s, (struct sockaddr*)&a, sizeof(a)) != 0 || listen(s, 1024) != 0) {
    MCCL_WARN("bind/listen on %s:%u failed: %s", ip ? ip : "*", port, strerror(errno));
    close(s);
    return mcclSystemError;
  }
  if (boundPort != nullptr) {
    socklen_t len = sizeof(a);
    getsockname(s, (struct sockaddr*)&a, &len);
    *boundPort = ntohs(a.sin_port);
  }
  *fd = s;
  return mcclSuccess;
}

mcclResult_t sockWaitReadable(int fd, int timeoutMs) {
  struct pollfd p = {fd, POLLIN, 0};
  for (;;) {
    int rc = poll(&p, 1, timeoutMs);
    if (rc > 0) return (p.revents & (POLLIN | POLLHUP | POLLERR)) ? mcclSuccess : mcclSystemError;
    if (rc == 0) return mcclInProgress;
    if (errno != EINTR) MCCLFAIL(mcclSystemError);
  }
}

mcclResult_t sockAccept(int listenFd, int timeoutMs, int* fd) {
  mcclResult_t rc = sockWaitReadable(listenFd, timeoutMs);
  if (rc != mcclSuccess) return rc;
  if (faultInject("accept")) MCCLFAIL(mcclSystemError);
  int s = accept4(listenFd, nullptr, nullptr, SOCK_CLOEXEC);
  if (s < 0) {
    if (errno == EINTR || errno == EAGAIN || errno == ECONNABORTED) return mcclInProgress;
    MCCLFAIL(mcclSystemError);
  }
  tuneStream(s);
  *fd = s;
  return mcclSuccess;
}

static mcclResult_t connectOnce(const struct sockaddr_in& a, int timeoutMs, int* fd) {
  int s = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (s < 0) MCCLFAIL(mcclSystemError);
  sockSetBuffers(s, (int)(mcclParamSocketBufKb() * 1024));
  int fl = fcntl(s, F_GETFL, 0);
  fcntl(s, F_SETFL, fl | O_NONBLOCK);
  int rc = connect(s, (const struct sockaddr*)&a, sizeof(a));
  if (rc != 0 && errno != EINPROGRESS) {
    close(s);
    return mcclInProgress;  // refused: worth a retry
  }
  if (rc != 0) {
    struct pollfd p = {s, POLLOUT, 0};
    int pr;
    do { pr = poll(&p, 1, timeoutMs); } while (pr < 0 && errno == EINTR);
    int err = 0;
    socklen_t len = sizeof(err);
    if (pr <= 0 || getsockopt(s, SOL_SOCKET, SO_ERROR, &err, &len) != 0 || err != 0) {
      close(s);
      return mcclInProgress;
    }
  }
  fcntl(s, F_SETFL, fl);
  tuneStream(s);
  *fd = s;
  return mcclSuccess;
}

mcclResult_t sockConnect(const char* ip, uint16_t port, int timeoutMs, int retries, int* fd) {
  struct sockaddr_in a;
  memset(&a, 0, sizeof(a));
  a.sin_family = AF_INET;
  a.sin_port = htons(port);
  if (inet_pton(AF_INET, ip, &a.sin_addr) != 1) MCCLFAIL(mcclInvalidArgument);
  if (faultInject("connect")) MCCLFAIL(mcclSystemError);
  for (int attempt = 0; attempt <= retries; ++attempt) {
    mcclResult_t rc = connectOnce(a, timeoutMs, fd);
    if (rc == mcclSuccess) return rc;
    if (rc != mcclInProgress) return rc;
    usleep(100 * 1000);
  }
  MCCL_WARN("connect to %s:%u gave up after %d attempts", ip, port, retries + 1);
  return mcclSystemError;
}

mcclResult_t sockSend(int fd, const void* buf, size_t bytes) {
  const char* p = static_cast<const char*>(buf);
  if (faultInject("send")) MCCLFAIL(mcclSystemError);
  while (bytes > 0) {
    ssize_t n = send(fd, p, bytes, MSG_NOSIGNAL);
    if (n > 0) { p += n; bytes -= (size_t)n; continue; }
    if (n < 0 && (errno == EINTR || errno == ENOBUFS || errno == ENOMEM)) continue;
    MCCL_TRACE("send failed: %s", n == 0 ? "closed" : strerror(errno));
    return mcclSystemError;
  }
  return mcclSuccess;
}

mcclResult_t sockRecv(int fd, void* buf, size_t bytes) {
  char* p = static_cast<char*>(buf);
  if (faultInject("recv")) MCCLFAIL(mcclSystemError);
  while (bytes > 0) {
    ssize_t n = recv(fd, p, bytes, 0);
    if (n > 0) { p += n; bytes -= (size_t)n; continue; }
    if (n < 0 && (errno == EINTR || errno == ENOBUFS || errno == ENOMEM)) continue;
    MCCL_TRACE("recv failed: %s", n == 0 ? "peer closed" : strerror(errno));
    return n == 0 ? mcclRemoteError : mcclSystemError;
  }
  return mcclSuccess;
}

void sockShutdown(int fd) { if (fd >= 0) shutdown(fd, SHUT_RDWR); }
void sockClose(int fd) { if (fd >= 0) close(fd); }

static socklen_t abstractAddr(const char* name, struct sockaddr_un* a) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  size_t len = strlen(name);
  if (len > sizeof(a->sun_path) - 2) len = sizeof(a->sun_path) - 2;
  memcpy(a->sun_path + 1, name, len);  // leading NUL = abstract namespace, nothing to unlink
  return (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + len);
}

mcclResult_t udsBind(const char* name, int* fd) {
  int s = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (s < 0) MCCLFAIL(mcclSystemError);
  struct sockaddr_un a;
  socklen_t len = abstractAddr(name, &a);
  if (bind(s, (struct sockaddr*)&a, len) != 0) {
    MCCL_WARN("uds bind %s failed: %s", name, strerror(errno));
    close(s);
    return mcclSystemError;
  }
  *fd = s;
  return mcclSuccess;
}

mcclResult_t udsSendFd(int fd, const char* name, int sendFd, const void* payload, size_t bytes) {
  struct sockaddr_un a;
  socklen_t alen = abstractAddr(name, &a);
  struct iovec iov = {const_cast<void*>(payload), bytes};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  struct msghdr m;
  memset(&m, 0, sizeof(m));
  m.msg_name = &a;
  m.msg_namelen = alen;
  m.msg_iov = &iov;
  m.msg_iovlen = 1;
  if (sendFd >= 0) {
    m.msg_control = ctrl;
    m.msg_controllen = sizeof(ctrl);
    struct cmsghdr* c = CMSG_FIRSTHDR(&m);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &sendFd, sizeof(int));
  }
  for (int attempt = 0; attempt < 300; ++attempt) {
    ssize_t n = sendmsg(fd, &m, MSG_NOSIGNAL);
    if (n == (ssize_t)bytes) return mcclSuccess;
    // The peer may not have bound its endpoint yet, or its queue is full: both clear by waiting.
    if (n < 0 && (errno == EINTR || errno == ECONNREFUSED || errno == ENOENT || errno == EAGAIN ||
                  errno == ENOBUFS)) {
      usleep(10 * 1000);
      continue;
    }
    MCCL_WARN("uds send to %s failed: %s", name, strerror(errno));
    return mcclSystemError;
  }
  return mcclSystemError;
}

mcclResult_t udsRecvFd(int fd, int timeoutMs, int* recvFd, void* payload, size_t bytes) {
  mcclResult_t rc = sockWaitReadable(fd, timeoutMs);
  if (rc != mcclSuccess) return rc;
  struct iovec iov = {payload, bytes};
  char ctrl[CMSG_SPACE(sizeof(int))];
  struct msghdr m;
  memset(&m, 0, sizeof(m));
  m.msg_iov = &iov;
  m.msg_iovlen = 1;
  m.msg_control = ctrl;
  m.msg_controllen = sizeof(ctrl);
  ssize_t n;
  do { n = recvmsg(fd, &m, MSG_CMSG_CLOEXEC); } while (n < 0 && errno == EINTR);
  if (n != (ssize_t)bytes) MCCLFAIL(mcclSystemError);
  *recvFd = -1;
  for (struct cmsghdr* c = CMSG_FIRSTHDR(&m); c != nullptr; c = CMSG_NXTHDR(&m, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(recvFd, CMSG_DATA(c), sizeof(int));
  }
  return mcclSuccess;
}

}  // namespace mccl
