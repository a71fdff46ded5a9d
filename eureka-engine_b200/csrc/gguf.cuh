// gguf.cuh -- a GGUF file mapped read-only and described as the engine's index text (gguf.cu).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <string>

struct GgufFile {
  int fd = -1;
  const uint8_t *map = nullptr;   // the whole file; tensor offsets in `index` are relative to it
  size_t size = 0;
  std::string index;              // "#cfg" lines and one line per tensor the path reads
  int nextn = 0;                  // MTP blocks the file holds after the trunk
};
int gguf_map(const char *path, GgufFile &g);   // 0, or -1 with llb_fail's message
void gguf_unmap(GgufFile &g);
