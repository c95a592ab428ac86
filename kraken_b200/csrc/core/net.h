// Request / reply transport of the multi-process CPU deployment, native part: framing, body
// compression, a client with timeouts and a threaded server.
//
// The reference's processes talk over ZeroMQ with a 13-byte header in front of every body
// (kraken/rpc/protocol.h:12-41), a server that hands each request to a worker thread and answers in
// the request's compression (kraken/rpc/station.cc:127-228, kraken/rpc/station.h:62-119) and a client
// whose calls time out after 5 s (kraken/rpc/indep_connecter.h:83-84).  Here the same shape runs on
// plain TCP sockets:
//
//   frame  = u32 body_len | u64 stamp (correlation id) | i32 type (request) or error code (reply) | u8 compress | body
//
// compress = 1 means the body is a Snappy stream (snappy_codec.h); the header is never compressed.
// What a body means (metadata + tensors) is the caller's business: this layer moves bytes.
#pragma once

#include <atomic>
#include <cstdint>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <utility>
#include <vector>

namespace kb {
namespace net {

constexpr uint8_t kCompressNone = 0;
constexpr uint8_t kCompressSnappy = 1;
constexpr uint32_t kMaxBody = 0xFFFFFFFFu;  // the length field is 32 bits

struct Frame {
  uint64_t stamp = 0;
  int32_t code = 0;  // RPC type in a request, error code in a reply
  uint8_t compress = kCompressNone;
  std::string body;  // as the application sent it (already uncompressed on the receiving side)
};

enum class RecvStatus { kOk, kClosed, kTimeout, kBadFrame };

// Sends one frame (compressing the body when `compress` says so).  False: the peer is gone.
bool SendFrame(int fd, uint64_t stamp, int32_t code, const std::string& body, uint8_t compress);
// Receives one frame.  timeout_ms < 0: no limit.  The limit covers the wait for the first byte and every
// later stall of the same frame.
RecvStatus RecvFrame(int fd, int timeout_ms, Frame* out);

// Client for one peer.  Call() is synchronous and serialised by a lock; replies to calls that timed out
// earlier are recognised by their stamp and dropped.
class Connecter {
 public:
  Connecter(const std::string& host, int port, int timeout_ms, uint8_t compress);
  ~Connecter();
  Connecter(const Connecter&) = delete;
  Connecter& operator=(const Connecter&) = delete;
  // (reply code, reply body).  Throws KrakenError: kTimeout when no reply arrives in time (timeout_ms <= 0:
  // the connecter's default), kConnection when the peer closed the connection or sent a broken frame.
  std::pair<int32_t, std::string> Call(uint32_t type, const std::string& body, int timeout_ms);
  void Close();

 private:
  int fd_ = -1;
  std::mutex mu_;
  uint64_t stamp_;
  int timeout_ms_;
  uint8_t compress_;
  std::string addr_;
};

// (reply code, reply body) for (request type, request body); runs on the connection's thread.
using Handler = std::function<std::pair<int32_t, std::string>(uint32_t, const std::string&)>;

// Threaded server: one thread accepts, one thread per connection reads requests and answers them in
// order; a successful reply travels in the compression of its request, an error reply uncompressed.
class Station {
 public:
  Station(const std::string& host, int port, Handler handler);  // binds and listens; port 0: any free port
  ~Station();
  Station(const Station&) = delete;
  Station& operator=(const Station&) = delete;
  int port() const { return port_; }
  void Start();
  // Closes the listener and every connection and waits for the threads.  Must not be called from a handler.
  void Stop();

 private:
  struct Shared;
  std::shared_ptr<Shared> st_;
  std::thread acceptor_;
  int port_ = 0;
  bool started_ = false;
};

}  // namespace net
}  // namespace kb
