// Host-side IO runtime: byte-range reads for safetensors, safetensors writer, uint16 token
// shard loader, BOS position finder, WAV (PCM16) and PPM writers.
//
// The reference keeps header parsing in Lean and lets the native side move bytes
// (cc/src/tyr.cpp:2525-2596 safetensors_read/write, :1771-1829 bin_file_token_count / load_u16_bin,
// :2600-2660 find_bos_positions, :2193-2296 save_ppm, :2298-2480 save_wav / wav_begin/append/
// finalize).  The same split is kept: Python validates the JSON header, these functions do the
// bulk work (parallel pread into pinned or pageable destination buffers).
#include <algorithm>
#include <cerrno>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

#define TYR_HOST_EXPORT extern "C" __attribute__((visibility("default")))

namespace {
thread_local std::string g_last_error;
int fail(const std::string& msg) {
  g_last_error = msg;
  return -1;
}
bool pread_all(int fd, void* dst, size_t len, off_t off) {
  char* p = static_cast<char*>(dst);
  while (len > 0) {
    ssize_t r = pread(fd, p, len, off);
    if (r < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    if (r == 0) return false;  // truncated
    p += r;
    off += r;
    len -= static_cast<size_t>(r);
  }
  return true;
}
}  // namespace

TYR_HOST_EXPORT const char* tyr_host_last_error() { return g_last_error.c_str(); }

TYR_HOST_EXPORT long long tyr_file_size(const char* path) {
  struct stat st;
  if (stat(path, &st) != 0) return fail(std::string("Failed to stat: ") + path);
  return static_cast<long long>(st.st_size);
}

// Reads [offset, offset+length) of `path` into dst, split over up to `threads` readers.
TYR_HOST_EXPORT int tyr_file_read_range(const char* path, long long offset, long long length, void* dst,
                                        int threads) {
  if (length < 0 || offset < 0) return fail("negative offset/length");
  int fd = open(path, O_RDONLY);
  if (fd < 0) return fail(std::string("Failed to open: ") + path);
  struct stat st;
  if (fstat(fd, &st) != 0 || offset + length > st.st_size) {
    close(fd);
    return fail("SafeTensors load error: failed to read tensor data (file truncated).");
  }
  bool ok = true;
  const long long kMinChunk = 8LL << 20;
  int n = threads > 1 ? static_cast<int>(std::min<long long>(threads, std::max<long long>(1, length / kMinChunk))) : 1;
  if (n <= 1) {
    ok = length == 0 || pread_all(fd, dst, static_cast<size_t>(length), offset);
  } else {
    std::vector<std::thread> pool;
    std::vector<char> oks(n, 1);
    long long per = (length + n - 1) / n;
    for (int i = 0; i < n; ++i) {
      long long o = per * i, l = std::min(per, length - o);
      if (l <= 0) break;
      pool.emplace_back([=, &oks] {
        oks[i] = pread_all(fd, static_cast<char*>(dst) + o, static_cast<size_t>(l), offset + o) ? 1 : 0;
      });
    }
    for (auto& t : pool) t.join();
    for (char c : oks) ok = ok && c;
  }
  close(fd);
  return ok ? 0 : fail("SafeTensors load error: failed to read tensor data (file truncated).");
}

// Writes: u64 header size, header bytes, then each tensor's bytes in order.
TYR_HOST_EXPORT int tyr_safetensors_write(const char* path, const char* header, long long header_len, int count,
                                          const void* const* ptrs, const long long* lens) {
  FILE* f = fopen(path, "wb");
  if (!f) return fail(std::string("Failed to open output safetensors file: ") + path);
  uint64_t hs = static_cast<uint64_t>(header_len);
  bool ok = fwrite(&hs, sizeof(hs), 1, f) == 1;
  ok = ok && (header_len == 0 || fwrite(header, 1, static_cast<size_t>(header_len), f) == static_cast<size_t>(header_len));
  for (int i = 0; ok && i < count; ++i)
    ok = lens[i] == 0 || fwrite(ptrs[i], 1, static_cast<size_t>(lens[i]), f) == static_cast<size_t>(lens[i]);
  ok = (fflush(f) == 0) && ok;
  ok = (fsync(fileno(f)) == 0) && ok;
  ok = (fclose(f) == 0) && ok;
  return ok ? 0 : fail(std::string("Failed to write safetensors file: ") + path);
}

// ------------------------------------------------------------------------------------------
// uint16 token shards (optional 256 x int32 header with magic 20240520, version 1, token count)
// ------------------------------------------------------------------------------------------
static const int32_t kShardMagic = 20240520;
static const long long kShardHeaderBytes = 256 * 4;

TYR_HOST_EXPORT int tyr_bin_token_count(const char* path, long long* count, long long* header_bytes) {
  long long size = tyr_file_size(path);
  if (size < 0) return -1;
  *header_bytes = 0;
  if (size >= kShardHeaderBytes) {
    int32_t head[3];
    if (tyr_file_read_range(path, 0, sizeof(head), head, 1) != 0) return -1;
    if (head[0] == kShardMagic) {
      *header_bytes = kShardHeaderBytes;
      long long declared = head[2];
      long long avail = (size - kShardHeaderBytes) / 2;
      if (declared < 0 || declared > avail) return fail("token shard header declares more tokens than the file holds");
      *count = declared;
      return 0;
    }
  }
  if (size % 2 != 0) return fail("token shard size is not a multiple of 2 bytes");
  *count = size / 2;
  return 0;
}

TYR_HOST_EXPORT int tyr_load_u16_bin(const char* path, long long start_token, long long n, long long* dst) {
  long long count = 0, hb = 0;
  if (tyr_bin_token_count(path, &count, &hb) != 0) return -1;
  if (start_token < 0 || n < 0 || start_token + n > count) return fail("token range outside the shard");
  std::vector<uint16_t> tmp(static_cast<size_t>(n));
  if (n > 0 && tyr_file_read_range(path, hb + start_token * 2, n * 2, tmp.data(), 4) != 0) return -1;
  for (long long i = 0; i < n; ++i) dst[i] = tmp[static_cast<size_t>(i)];
  return 0;
}

TYR_HOST_EXPORT long long tyr_find_bos(const long long* tokens, long long n, long long bos, long long* out,
                                       long long cap) {
  long long k = 0;
  for (long long i = 0; i < n; ++i)
    if (tokens[i] == bos) {
      if (k < cap) out[k] = i;
      ++k;
    }
  return k;
}

// ------------------------------------------------------------------------------------------
// PPM (P6) and WAV (PCM16 mono/multi-channel) writers
// ------------------------------------------------------------------------------------------
// rgb: float [3, H, W] in [0, 1] (clamped)
TYR_HOST_EXPORT int tyr_save_ppm(const char* path, const float* rgb, int H, int W) {
  if (H <= 0 || W <= 0) return fail("save_ppm: empty image");
  FILE* f = fopen(path, "wb");
  if (!f) return fail(std::string("Failed to open: ") + path);
  fprintf(f, "P6\n%d %d\n255\n", W, H);
  std::vector<unsigned char> row(static_cast<size_t>(W) * 3);
  const size_t plane = static_cast<size_t>(H) * W;
  bool ok = true;
  for (int y = 0; y < H && ok; ++y) {
    for (int x = 0; x < W; ++x)
      for (int c = 0; c < 3; ++c) {
        float v = rgb[c * plane + static_cast<size_t>(y) * W + x];
        v = std::min(1.f, std::max(0.f, v));
        row[static_cast<size_t>(x) * 3 + c] = static_cast<unsigned char>(std::lround(v * 255.f));
      }
    ok = fwrite(row.data(), 1, row.size(), f) == row.size();
  }
  ok = (fclose(f) == 0) && ok;
  return ok ? 0 : fail("save_ppm: write failed");
}

namespace {
void put_u32(unsigned char* p, uint32_t v) { p[0] = v & 255; p[1] = (v >> 8) & 255; p[2] = (v >> 16) & 255; p[3] = v >> 24; }
void put_u16(unsigned char* p, uint16_t v) { p[0] = v & 255; p[1] = v >> 8; }
void wav_header(unsigned char* h, uint32_t data_bytes, int sample_rate, int channels) {
  memcpy(h, "RIFF", 4); put_u32(h + 4, 36 + data_bytes); memcpy(h + 8, "WAVEfmt ", 8);
  put_u32(h + 16, 16); put_u16(h + 20, 1); put_u16(h + 22, static_cast<uint16_t>(channels));
  put_u32(h + 24, static_cast<uint32_t>(sample_rate));
  put_u32(h + 28, static_cast<uint32_t>(sample_rate) * channels * 2);
  put_u16(h + 32, static_cast<uint16_t>(channels * 2)); put_u16(h + 34, 16);
  memcpy(h + 36, "data", 4); put_u32(h + 40, data_bytes);
}
bool write_pcm16(FILE* f, const float* s, long long n) {
  std::vector<int16_t> buf(static_cast<size_t>(std::min<long long>(n, 1 << 16)));
  long long done = 0;
  while (done < n) {
    long long m = std::min<long long>(n - done, static_cast<long long>(buf.size()));
    for (long long i = 0; i < m; ++i) {
      float v = std::min(1.f, std::max(-1.f, s[done + i]));
      buf[static_cast<size_t>(i)] = static_cast<int16_t>(std::lround(v * 32767.f));
    }
    if (fwrite(buf.data(), 2, static_cast<size_t>(m), f) != static_cast<size_t>(m)) return false;
    done += m;
  }
  return true;
}
}  // namespace

TYR_HOST_EXPORT int tyr_save_wav(const char* path, const float* samples, long long n, int sample_rate, int channels) {
  FILE* f = fopen(path, "wb");
  if (!f) return fail(std::string("Failed to open: ") + path);
  unsigned char h[44];
  wav_header(h, static_cast<uint32_t>(n * 2), sample_rate, channels);
  bool ok = fwrite(h, 1, 44, f) == 44 && write_pcm16(f, samples, n);
  ok = (fclose(f) == 0) && ok;
  return ok ? 0 : fail("save_wav: write failed");
}

// streaming WAV: begin writes a placeholder header, append adds samples, finalize patches sizes
TYR_HOST_EXPORT int tyr_wav_begin(const char* path, int sample_rate, int channels) {
  FILE* f = fopen(path, "wb");
  if (!f) return fail(std::string("Failed to open: ") + path);
  unsigned char h[44];
  wav_header(h, 0, sample_rate, channels);
  bool ok = fwrite(h, 1, 44, f) == 44;
  ok = (fclose(f) == 0) && ok;
  return ok ? 0 : fail("wav_begin: write failed");
}
TYR_HOST_EXPORT int tyr_wav_append(const char* path, const float* samples, long long n) {
  FILE* f = fopen(path, "ab");
  if (!f) return fail(std::string("Failed to open: ") + path);
  bool ok = write_pcm16(f, samples, n);
  ok = (fclose(f) == 0) && ok;
  return ok ? 0 : fail("wav_append: write failed");
}
TYR_HOST_EXPORT int tyr_wav_finalize(const char* path, int sample_rate, int channels) {
  long long size = tyr_file_size(path);
  if (size < 44) return fail("wav_finalize: file has no header");
  FILE* f = fopen(path, "r+b");
  if (!f) return fail(std::string("Failed to open: ") + path);
  unsigned char h[44];
  wav_header(h, static_cast<uint32_t>(size - 44), sample_rate, channels);
  bool ok = fwrite(h, 1, 44, f) == 44;
  ok = (fclose(f) == 0) && ok;
  return ok ? 0 : fail("wav_finalize: write failed");
}
