#include "net.h"

#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <new>
#include <set>
#include <stdexcept>

#include "snappy_codec.h"
#include "types.h"

namespace kb {
namespace net {

namespace {

constexpr size_t kHeader = 4 + 8 + 4 + 1;  // body length + the 13-byte header

void PutLE(char* p, uint64_t v, int bytes) {
  for (int i = 0; i < bytes; ++i) p[i] = static_cast<char>((v >> (8 * i)) & 0xff);
}
uint64_t GetLE(const char* p, int bytes) {
  uint64_t v = 0;
  for (int i = 0; i < bytes; ++i) v |= static_cast<uint64_t>(static_cast<unsigned char>(p[i])) << (8 * i);
  return v;
}

bool WaitReadable(int fd, int timeout_ms, bool* timed_out) {
  for (;;) {
    pollfd p{fd, POLLIN, 0};
    const int r = ::poll(&p, 1, timeout_ms);
    if (r > 0) return true;
    if (r == 0) {
      *timed_out = true;
      return false;
    }
    if (errno != EINTR) return false;
  }
}

// Reads exactly n bytes.  kClosed also covers a peer that stops in the middle of a frame.
RecvStatus ReadAll(int fd, char* buf, size_t n, int timeout_ms) {
  while (n > 0) {
    if (timeout_ms >= 0) {
      bool timed_out = false;
      if (!WaitReadable(fd, timeout_ms, &timed_out)) return timed_out ? RecvStatus::kTimeout : RecvStatus::kClosed;
    }
    const ssize_t got = ::recv(fd, buf, n, 0);
    if (got < 0 && errno == EINTR) continue;
    if (got <= 0) return RecvStatus::kClosed;
    buf += got;
    n -= static_cast<size_t>(got);
  }
  return RecvStatus::kOk;
}

bool WriteAll(int fd, const char* a, size_t na, const char* b, size_t nb) {
  while (na + nb > 0) {
    iovec iov[2];
    int cnt = 0;
    if (na) iov[cnt++] = {const_cast<char*>(a), na};
    if (nb) iov[cnt++] = {const_cast<char*>(b), nb};
    msghdr msg{};
    msg.msg_iov = iov;
    msg.msg_iovlen = static_cast<size_t>(cnt);
    const ssize_t put = ::sendmsg(fd, &msg, MSG_NOSIGNAL);
    if (put < 0 && errno == EINTR) continue;
    if (put <= 0) return false;
    size_t left = static_cast<size_t>(put);
    const size_t from_a = left < na ? left : na;
    a += from_a;
    na -= from_a;
    left -= from_a;
    b += left;
    nb -= left;
  }
  return true;
}

void NoDelay(int fd) {
  int one = 1;
  ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}

}  // namespace

bool SendFrame(int fd, uint64_t stamp, int32_t code, const std::string& body, uint8_t compress) {
  std::string packed;
  const std::string* payload = &body;
  if (compress == kCompressSnappy) {
    snappy_codec::Compress(body.data(), body.size(), &packed);
    payload = &packed;
  }
  KB_CHECK(payload->size() <= kMaxBody, err::kSerializeRequest, "a frame body is limited to 4 GiB");
  char head[kHeader];
  PutLE(head, payload->size(), 4);
  PutLE(head + 4, stamp, 8);
  PutLE(head + 12, static_cast<uint32_t>(code), 4);
  head[16] = static_cast<char>(compress);
  return WriteAll(fd, head, kHeader, payload->data(), payload->size());
}

RecvStatus RecvFrame(int fd, int timeout_ms, Frame* out) {
  char head[kHeader];
  RecvStatus st = ReadAll(fd, head, kHeader, timeout_ms);
  if (st != RecvStatus::kOk) return st;
  const size_t n = static_cast<size_t>(GetLE(head, 4));
  out->stamp = GetLE(head + 4, 8);
  out->code = static_cast<int32_t>(static_cast<uint32_t>(GetLE(head + 12, 4)));
  out->compress = static_cast<uint8_t>(head[16]);
  if (out->compress != kCompressNone && out->compress != kCompressSnappy) return RecvStatus::kBadFrame;
  try {
    // the length comes off the wire: a peer that announces more than this host can hold is a broken peer,
    // not a reason to die
    // and the buffer grows with the bytes that really arrive (4 MiB at a time), not with the announcement
    std::string raw;
    for (size_t got = 0; got < n;) {
      const size_t step = std::min<size_t>(n - got, 4u << 20);
      raw.resize(got + step);
      st = ReadAll(fd, &raw[got], step, timeout_ms);
      if (st != RecvStatus::kOk) return st;
      got += step;
    }
    if (out->compress == kCompressNone) {
      out->body.swap(raw);
    } else if (!snappy_codec::Uncompress(raw.data(), raw.size(), &out->body)) {
      return RecvStatus::kBadFrame;
    }
  } catch (const std::bad_alloc&) {
    return RecvStatus::kBadFrame;
  } catch (const std::length_error&) {
    return RecvStatus::kBadFrame;
  }
  return RecvStatus::kOk;
}

// ------------------------------------------------------------------ client
Connecter::Connecter(const std::string& host, int port, int timeout_ms, uint8_t compress)
    : timeout_ms_(timeout_ms > 0 ? timeout_ms : 5000), compress_(compress), addr_(host + ":" + std::to_string(port)) {
  addrinfo hints{};
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  addrinfo* res = nullptr;
  const int rc = ::getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res);
  KB_CHECK(rc == 0 && res != nullptr, err::kConnection, "cannot resolve " + addr_);
  for (addrinfo* a = res; a != nullptr && fd_ < 0; a = a->ai_next) {
    const int fd = ::socket(a->ai_family, a->ai_socktype, a->ai_protocol);
    if (fd < 0) continue;
    if (::connect(fd, a->ai_addr, a->ai_addrlen) == 0) {
      fd_ = fd;
    } else {
      ::close(fd);
    }
  }
  ::freeaddrinfo(res);
  KB_CHECK(fd_ >= 0, err::kConnection, "cannot connect to " + addr_);
  NoDelay(fd_);
  stamp_ = static_cast<uint64_t>(
      std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::system_clock::now().time_since_epoch()).count());
}

Connecter::~Connecter() { Close(); }

void Connecter::Close() {
  std::lock_guard<std::mutex> g(mu_);
  if (fd_ >= 0) {
    ::shutdown(fd_, SHUT_RDWR);
    ::close(fd_);
    fd_ = -1;
  }
}

std::pair<int32_t, std::string> Connecter::Call(uint32_t type, const std::string& body, int timeout_ms) {
  std::lock_guard<std::mutex> g(mu_);
  KB_CHECK(fd_ >= 0, err::kConnection, "the connection to " + addr_ + " is closed");
  const uint64_t stamp = ++stamp_;
  KB_CHECK(SendFrame(fd_, stamp, static_cast<int32_t>(type), body, compress_), err::kConnection,
           addr_ + " closed the connection");
  const int limit = timeout_ms > 0 ? timeout_ms : timeout_ms_;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(limit);
  Frame f;
  for (;;) {
    const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - std::chrono::steady_clock::now()).count();
    const RecvStatus st = left > 0 ? RecvFrame(fd_, static_cast<int>(left), &f) : RecvStatus::kTimeout;
    if (st == RecvStatus::kTimeout)
      throw KrakenError(err::kTimeout, addr_ + " type " + std::to_string(type) + ": no reply within " +
                                           std::to_string(limit) + " ms");
    KB_CHECK(st == RecvStatus::kOk, err::kConnection,
             addr_ + (st == RecvStatus::kBadFrame ? " sent a broken frame" : " closed the connection"));
    if (f.stamp == stamp) break;  // replies to calls that timed out earlier are dropped
  }
  return {f.code, std::move(f.body)};
}

// ------------------------------------------------------------------ server
struct Station::Shared {
  Handler handler;
  int listen_fd = -1;
  std::atomic<bool> stopping{false};
  std::mutex mu;
  std::set<int> conns;               // open connection sockets
  std::vector<std::thread> threads;  // one per connection ever accepted
};

Station::Station(const std::string& host, int port, Handler handler) : st_(std::make_shared<Shared>()) {
  st_->handler = std::move(handler);
  const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  KB_CHECK(fd >= 0, err::kConnection, "cannot create a socket");
  int one = 1;
  ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (host.empty() || host == "0.0.0.0") {
    addr.sin_addr.s_addr = htonl(INADDR_ANY);
  } else if (::inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1) {
    ::close(fd);
    KB_CHECK(false, err::kBadArgument, "not an IPv4 address: " + host);
  }
  if (::bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(fd, 128) != 0) {
    const std::string why = std::strerror(errno);
    ::close(fd);
    KB_CHECK(false, err::kConnection, "cannot listen on port " + std::to_string(port) + ": " + why);
  }
  socklen_t len = sizeof(addr);
  ::getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &len);
  port_ = ntohs(addr.sin_port);
  st_->listen_fd = fd;
}

void Station::Start() {
  if (started_) return;
  started_ = true;
  std::shared_ptr<Shared> st = st_;
  acceptor_ = std::thread([st] {
    for (;;) {
      const int c = ::accept(st->listen_fd, nullptr, nullptr);
      if (c < 0) {
        if (errno == EINTR) continue;
        return;  // the listener was shut down
      }
      NoDelay(c);
      std::lock_guard<std::mutex> g(st->mu);
      if (st->stopping) {
        ::close(c);
        return;
      }
      st->conns.insert(c);
      st->threads.emplace_back([st, c] {
        try {
          Frame req;
          while (RecvFrame(c, -1, &req) == RecvStatus::kOk) {
            std::pair<int32_t, std::string> reply;
            try {
              reply = st->handler(static_cast<uint32_t>(req.code), req.body);
            } catch (const KrakenError& e) {
              reply = {e.code, e.what()};
            } catch (const std::exception& e) {  // a failing handler must not take the server down
              reply = {err::kUnknown, e.what()};
            }
            if (!SendFrame(c, req.stamp, reply.first, reply.second, reply.first == 0 ? req.compress : kCompressNone))
              break;
          }
        } catch (...) {
          // nothing may leave a connection's thread: the connection is dropped, the server stays
        }
        std::lock_guard<std::mutex> g2(st->mu);
        if (st->conns.erase(c)) ::close(c);
      });
    }
  });
}

void Station::Stop() {
  if (!st_) return;
  std::vector<std::thread> threads;
  {
    std::lock_guard<std::mutex> g(st_->mu);
    if (st_->stopping.exchange(true)) return;
    if (st_->listen_fd >= 0) ::shutdown(st_->listen_fd, SHUT_RDWR);
    for (int c : st_->conns) ::shutdown(c, SHUT_RDWR);  // their threads fall out of recv and close them
  }
  if (acceptor_.joinable()) acceptor_.join();
  {
    std::lock_guard<std::mutex> g(st_->mu);
    threads.swap(st_->threads);
  }
  for (auto& t : threads)
    if (t.joinable()) t.join();
  std::lock_guard<std::mutex> g(st_->mu);
  if (st_->listen_fd >= 0) {
    ::close(st_->listen_fd);
    st_->listen_fd = -1;
  }
}

Station::~Station() {
  // a station that is still serving is shut down; its threads are not waited for here (one of them may be
  // inside a handler that needs a lock the destroying thread holds): they own the shared state and end on
  // their own once their sockets are shut down
  if (!st_) return;
  bool was_running;
  {
    std::lock_guard<std::mutex> g(st_->mu);
    was_running = !st_->stopping.exchange(true);
    if (was_running) {
      if (st_->listen_fd >= 0) ::shutdown(st_->listen_fd, SHUT_RDWR);
      for (int c : st_->conns) ::shutdown(c, SHUT_RDWR);
    }
  }
  if (acceptor_.joinable()) {
    if (was_running) acceptor_.detach(); else acceptor_.join();
  }
  std::lock_guard<std::mutex> g(st_->mu);
  for (auto& t : st_->threads)
    if (t.joinable()) t.detach();
  st_->threads.clear();
  if (!started_ && st_->listen_fd >= 0) {
    ::close(st_->listen_fd);
    st_->listen_fd = -1;
  }
}

}  // namespace net
}  // namespace kb
