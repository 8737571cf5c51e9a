// Growable float ring buffer for streaming audio (the reference's cc/src/float_buffer.cpp:
// mk/size/rms/get/push/append/clear/to_array/keep_last), plus the media entry points that only
// exist on macOS in the reference and return an error everywhere else
// (cc/src/tyr_media_stub.cpp:16-44, apple_audio_input.mm:275-310, apple_audio_output.mm:198-216).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#define TYR_HOST_EXPORT extern "C" __attribute__((visibility("default")))

struct TyrFloatBuffer {
  std::vector<float> data;
};

TYR_HOST_EXPORT TyrFloatBuffer* tyr_float_buffer_new() { return new TyrFloatBuffer(); }
TYR_HOST_EXPORT void tyr_float_buffer_free(TyrFloatBuffer* b) { delete b; }
TYR_HOST_EXPORT long long tyr_float_buffer_size(const TyrFloatBuffer* b) { return static_cast<long long>(b->data.size()); }
TYR_HOST_EXPORT double tyr_float_buffer_rms(const TyrFloatBuffer* b) {
  if (b->data.empty()) return 0.0;
  double s = 0.0;
  for (float v : b->data) s += static_cast<double>(v) * v;
  return std::sqrt(s / static_cast<double>(b->data.size()));
}
TYR_HOST_EXPORT int tyr_float_buffer_get(const TyrFloatBuffer* b, long long i, float* out) {
  if (i < 0 || i >= static_cast<long long>(b->data.size())) return -1;
  *out = b->data[static_cast<size_t>(i)];
  return 0;
}
TYR_HOST_EXPORT void tyr_float_buffer_push(TyrFloatBuffer* b, float v) { b->data.push_back(v); }
TYR_HOST_EXPORT void tyr_float_buffer_append(TyrFloatBuffer* b, const float* src, long long n) {
  if (n > 0) b->data.insert(b->data.end(), src, src + n);
}
TYR_HOST_EXPORT void tyr_float_buffer_append_buffer(TyrFloatBuffer* b, const TyrFloatBuffer* other) {
  b->data.insert(b->data.end(), other->data.begin(), other->data.end());
}
TYR_HOST_EXPORT void tyr_float_buffer_clear(TyrFloatBuffer* b) { b->data.clear(); }
TYR_HOST_EXPORT void tyr_float_buffer_copy_out(const TyrFloatBuffer* b, float* dst) {
  if (!b->data.empty()) memcpy(dst, b->data.data(), b->data.size() * sizeof(float));
}
TYR_HOST_EXPORT void tyr_float_buffer_keep_last(TyrFloatBuffer* b, long long n) {
  if (n <= 0) { b->data.clear(); return; }
  if (static_cast<long long>(b->data.size()) > n) b->data.erase(b->data.begin(), b->data.end() - n);
}

// ---- macOS-only media paths: error stubs on Linux ------------------------------------------
static const char* kAppleOnly = "Apple media path requires macOS build";
TYR_HOST_EXPORT const char* tyr_media_load_image_patchified(const char*) { return kAppleOnly; }
TYR_HOST_EXPORT const char* tyr_media_load_video_patchified(const char*) { return kAppleOnly; }
TYR_HOST_EXPORT const char* tyr_media_load_image_patch_grid_gemma4(const char*) { return kAppleOnly; }
TYR_HOST_EXPORT const char* tyr_audio_input_start() { return "Apple audio input requires macOS build"; }
TYR_HOST_EXPORT const char* tyr_audio_output_beep() { return "Apple audio output requires macOS build"; }
TYR_HOST_EXPORT int tyr_apple_mps_is_available() { return 0; }
