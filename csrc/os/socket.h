// Blocking TCP helpers with deadlines, plus an AF_UNIX datagram channel that carries file descriptors
// (cuMem POSIX handles) between ranks of one host.
// Parity: src/socket.h:11-22, src/socket.cc:19-173 of the reference (listen/accept/connect/send/recv with
// poll-based timeouts and EINTR/ENOBUFS retry); the fd-passing half has no counterpart there.
#pragma once

#include <cstddef>
#include <cstdint>

#include "../core/core.h"

namespace mccl {

// Listen on `ip` (nullptr = any) and `port` (0 = ephemeral).  Socket buffers are set on the listener so
// accepted sockets inherit them.
mcclResult_t sockListen(const char* ip, uint16_t port, int* fd, uint16_t* boundPort);
// Accept with a timeout in ms (<0 = forever).  mcclInProgress on timeout.
mcclResult_t sockAccept(int listenFd, int timeoutMs, int* fd);
// Non-blocking connect with a per-attempt timeout, retried `retries` times 100 ms apart.
mcclResult_t sockConnect(const char* ip, uint16_t port, int timeoutMs, int retries, int* fd);
mcclResult_t sockSend(int fd, const void* buf, size_t bytes);
mcclResult_t sockRecv(int fd, void* buf, size_t bytes);
// Wait until `fd` is readable; mcclInProgress on timeout.
mcclResult_t sockWaitReadable(int fd, int timeoutMs);
void         sockSetDeadline(int fd, int seconds);   // SO_SNDTIMEO/SO_RCVTIMEO, 0 = none
void         sockSetBuffers(int fd, int bytes);      // SO_SNDBUF/SO_RCVBUF
void         sockSetKeepalive(int fd, int idleSec);
void         sockShutdown(int fd);                   // unblock parked threads, keep the fd
void         sockClose(int fd);
MCCL_PARAM(SocketBufKb);

// AF_UNIX datagram endpoint bound to an abstract name.
mcclResult_t udsBind(const char* name, int* fd);
// Send `payload` plus (optionally, sendFd >= 0) one file descriptor to the endpoint called `name`.
mcclResult_t udsSendFd(int fd, const char* name, int sendFd, const void* payload, size_t bytes);
// Receive one datagram; *recvFd = -1 if it carried no descriptor.  mcclInProgress on timeout.
mcclResult_t udsRecvFd(int fd, int timeoutMs, int* recvFd, void* payload, size_t bytes);

}  // namespace mccl
