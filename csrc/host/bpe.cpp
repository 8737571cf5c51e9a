// Byte-pair encoding in native code: chunk encoding against a merge table and merge training over weighted words.
//
// The tokenizer's pre-tokenisation (the GPT-4 split pattern) and its file format stay in Python
// (tyr_b200/tokenizer/bpe.py); what runs here are the two loops that dominate tokenising a corpus and training a vocabulary.
// Semantics match the Python implementation exactly, so either side can stand in for the other:
//   * encode: start from byte tokens; repeatedly take the adjacent pair with the lowest merge rank and replace ALL its
//     occurrences left to right; stop when no adjacent pair has a rank.
//   * train: counts of adjacent pairs (overlapping occurrences count) weighted by word frequency; each step merges the pair
//     with the highest count, ties broken by the smaller left id and then the smaller right id; stops when the requested
//     number of merges is reached or no pair has a positive count.
// The reference implements both in Lean (Tyr/Tokenizer/Encode.lean, Tyr/Tokenizer/Training.lean:211).
#include <algorithm>
#include <cstdint>
#include <queue>
#include <thread>
#include <tuple>
#include <unordered_map>
#include <vector>

#define TYR_HOST_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

inline uint64_t pair_key(int32_t a, int32_t b) {
  return (static_cast<uint64_t>(static_cast<uint32_t>(a)) << 32) | static_cast<uint32_t>(b);
}

struct MergeInfo {
  int32_t rank;
  int32_t result;
};

}  // namespace

struct TyrBpe {
  std::unordered_map<uint64_t, MergeInfo> merges;
  int32_t byte_to_id[256];
};

// left / right / result: the merge rules in rank order; byte_to_id: token id of every single byte (-1 where the vocabulary
// has none).  Returns nullptr on a null argument.
TYR_HOST_EXPORT TyrBpe* tyr_bpe_new(const int32_t* left, const int32_t* right, const int32_t* result, long long n_merges,
                                    const int32_t* byte_to_id) {
  if (byte_to_id == nullptr || n_merges < 0 || (n_merges > 0 && (left == nullptr || right == nullptr || result == nullptr)))
    return nullptr;
  TyrBpe* t = new TyrBpe();
  t->merges.reserve(static_cast<size_t>(n_merges) * 2 + 16);
  for (long long i = 0; i < n_merges; ++i)
    t->merges.emplace(pair_key(left[i], right[i]), MergeInfo{static_cast<int32_t>(i), result[i]});   // first rule of a pair wins
  for (int i = 0; i < 256; ++i) t->byte_to_id[i] = byte_to_id[i];
  return t;
}

TYR_HOST_EXPORT void tyr_bpe_free(TyrBpe* t) { delete t; }

namespace {

// Encodes bytes[b0, b1) into out (room for b1 - b0 ids); returns the number of ids, or -1 when a byte has no token.
long long encode_chunk(const TyrBpe& t, const uint8_t* bytes, long long b0, long long b1, int32_t* out) {
  long long n = b1 - b0;
  for (long long i = 0; i < n; ++i) {
    const int32_t id = t.byte_to_id[bytes[b0 + i]];
    if (id < 0) return -1;
    out[i] = id;
  }
  while (n >= 2) {
    int32_t best_rank = INT32_MAX, best_result = 0, best_l = 0, best_r = 0;
    for (long long i = 0; i + 1 < n; ++i) {
      auto it = t.merges.find(pair_key(out[i], out[i + 1]));
      if (it != t.merges.end() && it->second.rank < best_rank) {
        best_rank = it->second.rank;
        best_result = it->second.result;
        best_l = out[i];
        best_r = out[i + 1];
      }
    }
    if (best_rank == INT32_MAX) break;
    long long w = 0;
    for (long long i = 0; i < n;) {
      if (i + 1 < n && out[i] == best_l && out[i + 1] == best_r) {
        out[w++] = best_result;
        i += 2;
      } else {
        out[w++] = out[i++];
      }
    }
    n = w;
  }
  return n;
}

}  // namespace

// Chunk i is bytes[offsets[i], offsets[i + 1]).  Its ids are written to out[offsets[i] ...] (a chunk never yields more ids
// than it has bytes) and their number to counts[i]; the caller compacts.  `threads` <= 1 runs on the calling thread.
// Returns 0, -1 on a null argument, or 1 + the index of the first chunk that holds a byte without a token.
TYR_HOST_EXPORT long long tyr_bpe_encode_chunks(const TyrBpe* t, const uint8_t* bytes, const long long* offsets, long long n_chunks,
                                                int32_t* out, long long* counts, int threads) {
  if (t == nullptr || offsets == nullptr || counts == nullptr || n_chunks < 0 || (n_chunks > 0 && (bytes == nullptr || out == nullptr)))
    return -1;
  std::vector<long long> bad(static_cast<size_t>(threads > 1 ? threads : 1), -1);
  auto work = [&](int tid, int nthreads) {
    for (long long i = tid; i < n_chunks; i += nthreads) {
      const long long c = encode_chunk(*t, bytes, offsets[i], offsets[i + 1], out + offsets[i]);
      if (c < 0) {
        counts[i] = 0;
        if (bad[static_cast<size_t>(tid)] < 0 || i < bad[static_cast<size_t>(tid)]) bad[static_cast<size_t>(tid)] = i;
      } else {
        counts[i] = c;
      }
    }
  };
  if (threads <= 1 || n_chunks < 256) {
    work(0, 1);
  } else {
    std::vector<std::thread> pool;
    for (int k = 0; k < threads; ++k) pool.emplace_back(work, k, threads);
    for (auto& th : pool) th.join();
  }
  long long first = -1;
  for (long long b : bad)
    if (b >= 0 && (first < 0 || b < first)) first = b;
  return first < 0 ? 0 : 1 + first;
}

// The same encoding with the ids of all chunks written back to back at the start of `out` (room for offsets[n_chunks] ids);
// returns their number, -1 on a null argument, or -(2 + i) when chunk i holds a byte without a token.
TYR_HOST_EXPORT long long tyr_bpe_encode_concat(const TyrBpe* t, const uint8_t* bytes, const long long* offsets, long long n_chunks,
                                                int32_t* out, int threads) {
  if (t == nullptr || offsets == nullptr || n_chunks < 0 || (n_chunks > 0 && (bytes == nullptr || out == nullptr))) return -1;
  std::vector<long long> counts(static_cast<size_t>(n_chunks > 0 ? n_chunks : 1));
  const long long rc = tyr_bpe_encode_chunks(t, bytes, offsets, n_chunks, out, counts.data(), threads);
  if (rc < 0) return -1;
  if (rc > 0) return -(1 + rc);
  long long w = 0;
  for (long long i = 0; i < n_chunks; ++i) {
    const long long c = counts[static_cast<size_t>(i)];
    if (w != offsets[i]) std::copy(out + offsets[i], out + offsets[i] + c, out + w);     // moves left: ranges never clobber
    w += c;
  }
  return w;
}

// Word i is the byte string bytes[offsets[i], offsets[i + 1]) seen freqs[i] times.  New token ids start at `first_id`
// (256 for a byte-level vocabulary whose byte b has id b).  Writes up to max_merges rules to out_left / out_right (rule j
// creates id first_id + j) and returns how many were made, or -1 on a bad argument.
TYR_HOST_EXPORT long long tyr_bpe_train(const uint8_t* bytes, const long long* offsets, const long long* freqs, long long n_words,
                                        long long max_merges, int32_t first_id, int32_t* out_left, int32_t* out_right) {
  if (offsets == nullptr || freqs == nullptr || n_words < 0 || max_merges < 0 || (max_merges > 0 && (out_left == nullptr || out_right == nullptr)))
    return -1;
  std::vector<std::vector<int32_t>> seqs(static_cast<size_t>(n_words));
  std::unordered_map<uint64_t, long long> count;
  std::unordered_map<uint64_t, std::vector<int32_t>> where;
  for (long long w = 0; w < n_words; ++w) {
    auto& s = seqs[static_cast<size_t>(w)];
    s.reserve(static_cast<size_t>(offsets[w + 1] - offsets[w]));
    for (long long i = offsets[w]; i < offsets[w + 1]; ++i) s.push_back(bytes[i]);
    for (size_t i = 0; i + 1 < s.size(); ++i) {
      const uint64_t k = pair_key(s[i], s[i + 1]);
      count[k] += freqs[w];
      auto& v = where[k];
      if (v.empty() || v.back() != static_cast<int32_t>(w)) v.push_back(static_cast<int32_t>(w));
    }
  }
  // max-heap on (count, smaller left, smaller right); entries go stale when a count changes and are skipped when popped
  using Entry = std::tuple<long long, int32_t, int32_t>;          // (count, -left, -right): std::less gives the order wanted
  std::priority_queue<Entry> heap;
  for (const auto& kv : count)
    if (kv.second > 0) heap.emplace(kv.second, -static_cast<int32_t>(kv.first >> 32), -static_cast<int32_t>(kv.first & 0xffffffffu));
  std::vector<int32_t> stamp(static_cast<size_t>(n_words), -1);
  std::vector<uint64_t> touched;
  long long made = 0;
  while (made < max_merges && !heap.empty()) {
    const Entry top = heap.top();
    heap.pop();
    const int32_t a = -std::get<1>(top), b = -std::get<2>(top);
    const uint64_t key = pair_key(a, b);
    auto cit = count.find(key);
    if (cit == count.end() || cit->second != std::get<0>(top)) continue;      // stale
    if (cit->second <= 0) break;
    const int32_t new_id = first_id + static_cast<int32_t>(made);
    out_left[made] = a;
    out_right[made] = b;
    touched.clear();
    auto wit = where.find(key);
    if (wit != where.end()) {
      std::vector<int32_t> words;
      words.swap(wit->second);
      where.erase(wit);
      for (int32_t w : words) {
        if (stamp[static_cast<size_t>(w)] == static_cast<int32_t>(made)) continue;     // listed twice
        stamp[static_cast<size_t>(w)] = static_cast<int32_t>(made);
        auto& s = seqs[static_cast<size_t>(w)];
        const long long f = freqs[w];
        bool has = false;
        for (size_t i = 0; i + 1 < s.size(); ++i)
          if (s[i] == a && s[i + 1] == b) { has = true; break; }
        if (!has) continue;                                        // the word lost the pair in an earlier merge
        for (size_t i = 0; i + 1 < s.size(); ++i) {
          const uint64_t k = pair_key(s[i], s[i + 1]);
          count[k] -= f;
          touched.push_back(k);
        }
        size_t wr = 0;
        for (size_t i = 0; i < s.size();) {
          if (i + 1 < s.size() && s[i] == a && s[i + 1] == b) {
            s[wr++] = new_id;
            i += 2;
          } else {
            s[wr++] = s[i++];
          }
        }
        s.resize(wr);
        for (size_t i = 0; i + 1 < s.size(); ++i) {
          const uint64_t k = pair_key(s[i], s[i + 1]);
          count[k] += f;
          touched.push_back(k);
          auto& v = where[k];
          if (v.empty() || v.back() != w) v.push_back(w);
        }
      }
    }
    std::sort(touched.begin(), touched.end());
    touched.erase(std::unique(touched.begin(), touched.end()), touched.end());
    for (uint64_t k : touched) {
      auto it = count.find(k);
      if (it == count.end()) continue;
      if (it->second <= 0) {
        count.erase(it);
      } else {
        heap.emplace(it->second, -static_cast<int32_t>(k >> 32), -static_cast<int32_t>(k & 0xffffffffu));
      }
    }
    count.erase(key);                                              // every occurrence is gone
    ++made;
  }
  return made;
}
