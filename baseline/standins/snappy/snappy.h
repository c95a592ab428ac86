// Stand-in for the two snappy 1.1.9 entry points the reference calls (kraken/common/compress.h:32,83;
// kraken/rpc/indep_connecter.cc:141).  The byte stream is the public snappy block format (varint length,
// then literal / copy elements), produced by an independently written hash-match compressor over 64 KiB
// blocks, so the reference does comparable CPU work per message to what it does with the real library.
#ifndef KRAKEN_BASELINE_SNAPPY_H_
#define KRAKEN_BASELINE_SNAPPY_H_

#include <stddef.h>

#include "snappy-sinksource.h"

namespace snappy {

// Compresses everything the source holds; returns the number of bytes appended to the sink.
size_t Compress(Source* reader, Sink* writer);

// Decompresses a stream made by Compress (or by snappy itself); false if the stream is malformed.
bool Uncompress(Source* compressed, Sink* uncompressed);

size_t MaxCompressedLength(size_t source_bytes);

}  // namespace snappy

#endif
