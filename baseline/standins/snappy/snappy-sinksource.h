// Byte source / sink interfaces with the signatures of snappy 1.1.9's snappy-sinksource.h, which the
// reference subclasses (kraken/common/snappy.h:9-72).  Part of the offline stand-in for the snappy
// library; written from the public interface, not copied from snappy.
#ifndef KRAKEN_BASELINE_SNAPPY_SINKSOURCE_H_
#define KRAKEN_BASELINE_SNAPPY_SINKSOURCE_H_

#include <stddef.h>

namespace snappy {

class Sink {
public:
  Sink() {}
  virtual ~Sink();
  virtual void Append(const char* bytes, size_t n) = 0;
  virtual char* GetAppendBuffer(size_t length, char* scratch);
  virtual void AppendAndTakeOwnership(char* bytes, size_t n, void (*deleter)(void*, const char*, size_t),
                                      void* deleter_arg);
  virtual char* GetAppendBufferVariable(size_t min_size, size_t desired_size_hint, char* scratch,
                                        size_t scratch_size, size_t* allocated_size);

private:
  Sink(const Sink&);
  void operator=(const Sink&);
};

class Source {
public:
  Source() {}
  virtual ~Source();
  virtual size_t Available() const = 0;
  virtual const char* Peek(size_t* len) = 0;
  virtual void Skip(size_t n) = 0;

private:
  Source(const Source&);
  void operator=(const Source&);
};

}  // namespace snappy

#endif
