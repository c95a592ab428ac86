/* Declarations of the ZeroMQ 4.x C API entry points that the benchmark's reference build calls
   (kraken/rpc/*.cc, kraken/common/zmq_buffer.cc), written from the public API documentation so that
   the reference can be compiled offline and linked against the libzmq shared library that ships inside
   the pyzmq wheel.  Only what the reference uses is declared. */
#ifndef KRAKEN_BASELINE_ZMQ_H_
#define KRAKEN_BASELINE_ZMQ_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZMQ_VERSION_MAJOR 4
#define ZMQ_VERSION_MINOR 3

/* socket types */
#define ZMQ_DEALER 5
#define ZMQ_ROUTER 6
/* socket options */
#define ZMQ_RCVMORE 13
/* send / receive flags */
#define ZMQ_DONTWAIT 1
#define ZMQ_SNDMORE 2
/* poll events */
#define ZMQ_POLLIN 1
#define ZMQ_POLLOUT 2
#define ZMQ_POLLERR 4

typedef int zmq_fd_t;

/* An opaque 64-byte message handle, pointer aligned (the layout every 4.x release has kept). */
typedef struct zmq_msg_t {
  unsigned char _[64] __attribute__((aligned(sizeof(void *))));
} zmq_msg_t;

typedef void(zmq_free_fn)(void *data_, void *hint_);

typedef struct zmq_pollitem_t {
  void *socket;
  zmq_fd_t fd;
  short events;
  short revents;
} zmq_pollitem_t;

int zmq_errno(void);
const char *zmq_strerror(int errnum_);

void *zmq_ctx_new(void);
int zmq_ctx_term(void *context_);
int zmq_term(void *context_);

void *zmq_socket(void *context_, int type_);
int zmq_close(void *s_);
int zmq_setsockopt(void *s_, int option_, const void *optval_, size_t optvallen_);
int zmq_getsockopt(void *s_, int option_, void *optval_, size_t *optvallen_);
int zmq_bind(void *s_, const char *addr_);
int zmq_connect(void *s_, const char *addr_);

int zmq_msg_init(zmq_msg_t *msg_);
int zmq_msg_init_size(zmq_msg_t *msg_, size_t size_);
int zmq_msg_init_data(zmq_msg_t *msg_, void *data_, size_t size_, zmq_free_fn *ffn_, void *hint_);
int zmq_msg_send(zmq_msg_t *msg_, void *s_, int flags_);
int zmq_msg_recv(zmq_msg_t *msg_, void *s_, int flags_);
int zmq_msg_close(zmq_msg_t *msg_);
int zmq_msg_move(zmq_msg_t *dest_, zmq_msg_t *src_);
int zmq_msg_copy(zmq_msg_t *dest_, zmq_msg_t *src_);
void *zmq_msg_data(zmq_msg_t *msg_);
size_t zmq_msg_size(const zmq_msg_t *msg_);
int zmq_msg_more(const zmq_msg_t *msg_);

int zmq_poll(zmq_pollitem_t *items_, int nitems_, long timeout_);
int zmq_proxy(void *frontend_, void *backend_, void *capture_);

#ifdef __cplusplus
}
#endif

#endif
