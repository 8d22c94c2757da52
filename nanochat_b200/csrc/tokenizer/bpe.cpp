// Byte-level BPE: trainer, encoder and the best-fit row packer, exposed to Python as `_tok`.
//
//   train_bpe(iterator, vocab_size) -> [(bytes, rank)]   streams texts from a Python iterator in
//        batches, splits and counts words on a thread pool (GIL released), then merges the most
//        frequent adjacent pair until `vocab_size` tokens exist. Pair counts are maintained
//        incrementally (only words containing the merged pair are touched) with a lazy max-heap.
//        Ties break toward the smaller (left id, right id) pair, so results are deterministic.
//   Encoder(token_bytes, ranks)   rank table; encode_ordinary / encode_ordinary_batch(num_threads)
//        split with the scanner and merge lowest-rank adjacent pairs inside each piece.
//   BestFitPacker(row_capacity, buffer_size)   packs token documents into fixed-length rows: largest
//        document that fits first, crop the shortest when none fits (oldest wins ties).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <functional>
#include <queue>
#include <set>
#include <string>
#include <string_view>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "scanner.h"

namespace py = pybind11;

namespace {

struct PairHash {
  size_t operator()(const std::pair<int, int>& p) const {
    return std::hash<uint64_t>()((static_cast<uint64_t>(static_cast<uint32_t>(p.first)) << 32) |
                                 static_cast<uint32_t>(p.second));
  }
};
using Pair = std::pair<int, int>;

void parallel_for(size_t n, int threads, const std::function<void(size_t, size_t, int)>& fn) {
  threads = std::max(1, std::min<int>(threads, static_cast<int>(n)));
  if (threads == 1) { fn(0, n, 0); return; }
  std::vector<std::thread> pool;
  const size_t per = (n + threads - 1) / threads;
  for (int t = 0; t < threads; ++t) {
    const size_t lo = t * per, hi = std::min(n, lo + per);
    if (lo >= hi) break;
    pool.emplace_back(fn, lo, hi, t);
  }
  for (auto& th : pool) th.join();
}

// ------------------------------------------------------------------------------ trainer
using WordCounts = std::unordered_map<std::string, long long>;

// Counts the pre-split words of a batch. Threads take texts from a shared counter (documents differ in length by
// orders of magnitude, so a static split leaves most threads idle), count into private maps keyed by views into the
// batch (no allocation per occurrence), and the maps are folded into `total`, copying a key only when it is new.
void count_words(const std::vector<std::string>& texts, int threads, WordCounts& total) {
  const int nt = std::max(1, std::min<int>(threads, static_cast<int>(texts.size())));
  using ViewCounts = std::unordered_map<std::string_view, long long>;
  std::vector<ViewCounts> partial(nt);
  std::atomic<size_t> next{0};
  auto work = [&](int t) {
    std::vector<std::pair<uint32_t, uint32_t>> pieces;
    ViewCounts& mine = partial[t];
    for (;;) {
      const size_t i = next.fetch_add(1);
      if (i >= texts.size()) return;
      pieces.clear();
      tok::split(texts[i], pieces);
      const char* base = texts[i].data();
      for (auto& pc : pieces) mine[std::string_view(base + pc.first, pc.second - pc.first)] += 1;
    }
  };
  if (nt == 1) {
    work(0);
  } else {
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) pool.emplace_back(work, t);
    for (auto& th : pool) th.join();
  }
  for (auto& m : partial)
    for (auto& kv : m) {
      auto f = total.find(std::string(kv.first));
      if (f == total.end()) total.emplace(std::string(kv.first), kv.second);
      else f->second += kv.second;
    }
}

std::vector<std::pair<py::bytes, int>> train_bpe(py::iterator it, int vocab_size, int threads) {
  if (vocab_size < 256) throw std::invalid_argument("vocab_size must be at least 256");
  WordCounts words;
  {
    std::vector<std::string> batch;
    size_t batch_bytes = 0;
    auto flush = [&]() {
      if (batch.empty()) return;
      py::gil_scoped_release nogil;
      count_words(batch, threads, words);
      batch.clear();
      batch_bytes = 0;
    };
    for (auto item : it) {
      batch.push_back(item.cast<std::string>());
      batch_bytes += batch.back().size();
      if (batch_bytes > (32u << 20)) flush();
    }
    flush();
  }
  std::vector<std::string> token_bytes(256);
  for (int b = 0; b < 256; ++b) token_bytes[b] = std::string(1, static_cast<char>(b));
  {
    py::gil_scoped_release nogil;
    // deterministic word order
    std::vector<std::pair<std::string, long long>> ordered(words.begin(), words.end());
    std::sort(ordered.begin(), ordered.end());
    std::vector<std::vector<int>> seqs(ordered.size());
    std::vector<long long> counts(ordered.size());
    for (size_t w = 0; w < ordered.size(); ++w) {
      counts[w] = ordered[w].second;
      seqs[w].reserve(ordered[w].first.size());
      for (unsigned char ch : ordered[w].first) seqs[w].push_back(ch);
    }
    std::unordered_map<Pair, long long, PairHash> pair_count;
    std::unordered_map<Pair, std::unordered_set<int>, PairHash> where;
    for (size_t w = 0; w < seqs.size(); ++w)
      for (size_t k = 0; k + 1 < seqs[w].size(); ++k) {
        const Pair p{seqs[w][k], seqs[w][k + 1]};
        pair_count[p] += counts[w];
        where[p].insert(static_cast<int>(w));
      }
    // max-heap on (count, smaller pair first)
    struct Entry { long long count; Pair pair; };
    auto worse = [](const Entry& a, const Entry& b) {
      if (a.count != b.count) return a.count < b.count;
      return a.pair > b.pair;
    };
    std::priority_queue<Entry, std::vector<Entry>, decltype(worse)> heap(worse);
    for (auto& kv : pair_count) heap.push({kv.second, kv.first});
    while (static_cast<int>(token_bytes.size()) < vocab_size && !heap.empty()) {
      const Entry top = heap.top();
      heap.pop();
      auto pc = pair_count.find(top.pair);
      if (pc == pair_count.end() || pc->second != top.count) continue;   // stale entry
      if (top.count <= 0) break;
      const int new_id = static_cast<int>(token_bytes.size());
      token_bytes.push_back(token_bytes[top.pair.first] + token_bytes[top.pair.second]);
      std::unordered_set<Pair, PairHash> touched;
      std::vector<int> users(where[top.pair].begin(), where[top.pair].end());
      std::sort(users.begin(), users.end());
      for (int w : users) {
        auto& s = seqs[w];
        const long long cnt = counts[w];
        // remove this word's contribution, rewrite it, add the contribution back
        for (size_t k = 0; k + 1 < s.size(); ++k) {
          const Pair p{s[k], s[k + 1]};
          pair_count[p] -= cnt;
          touched.insert(p);
        }
        std::vector<int> merged;
        merged.reserve(s.size());
        for (size_t k = 0; k < s.size();) {
          if (k + 1 < s.size() && s[k] == top.pair.first && s[k + 1] == top.pair.second) {
            merged.push_back(new_id);
            k += 2;
          } else {
            merged.push_back(s[k]);
            k += 1;
          }
        }
        s.swap(merged);
        for (size_t k = 0; k + 1 < s.size(); ++k) {
          const Pair p{s[k], s[k + 1]};
          pair_count[p] += cnt;
          where[p].insert(w);
          touched.insert(p);
        }
      }
      where.erase(top.pair);
      pair_count.erase(top.pair);
      for (const Pair& p : touched) {
        auto f = pair_count.find(p);
        if (f == pair_count.end()) continue;
        if (f->second <= 0) { pair_count.erase(f); continue; }
        heap.push({f->second, p});
      }
    }
  }
  std::vector<std::pair<py::bytes, int>> out;
  out.reserve(token_bytes.size());
  for (size_t i = 0; i < token_bytes.size(); ++i) out.emplace_back(py::bytes(token_bytes[i]), static_cast<int>(i));
  return out;
}

// ------------------------------------------------------------------------------ encoder
class Encoder {
 public:
  Encoder(const std::vector<std::string>& tokens, const std::vector<int>& ranks) {
    table_.reserve(tokens.size() * 2);
    for (size_t i = 0; i < tokens.size(); ++i) table_.emplace(tokens[i], ranks[i]);
  }

  void encode_into(std::string_view text, std::vector<int>& out) const {
    std::vector<std::pair<uint32_t, uint32_t>> pieces;
    tok::split(text, pieces);
    std::string key;
    for (auto& pc : pieces) encode_piece(text.substr(pc.first, pc.second - pc.first), out, key);
  }

  std::vector<int> encode_ordinary(const std::string& text) const {
    std::vector<int> out;
    py::gil_scoped_release nogil;
    encode_into(text, out);
    return out;
  }

  std::vector<std::vector<int>> encode_ordinary_batch(const std::vector<std::string>& texts, int num_threads) const {
    std::vector<std::vector<int>> out(texts.size());
    py::gil_scoped_release nogil;
    std::atomic<size_t> next{0};
    const int nt = std::max(1, std::min<int>(num_threads, static_cast<int>(texts.size())));
    auto work = [&]() {
      for (;;) {
        const size_t i = next.fetch_add(1);
        if (i >= texts.size()) return;
        encode_into(texts[i], out[i]);
      }
    };
    if (nt == 1) { work(); return out; }
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) pool.emplace_back(work);
    for (auto& th : pool) th.join();
    return out;
  }

 private:
  int rank_of(const std::string& key) const {
    auto f = table_.find(key);
    return f == table_.end() ? -1 : f->second;
  }

  // Lowest-rank-first merging inside one piece. parts[k] = start offset of part k.
  void encode_piece(std::string_view piece, std::vector<int>& out, std::string& key) const {
    key.assign(piece);
    int r = rank_of(key);
    if (r >= 0) { out.push_back(r); return; }
    const size_t n = piece.size();
    std::vector<uint32_t> starts(n + 1);
    for (size_t k = 0; k <= n; ++k) starts[k] = static_cast<uint32_t>(k);
    auto pair_rank = [&](size_t k) -> int {   // rank of parts k and k+1 joined
      if (k + 2 >= starts.size()) return -1;
      key.assign(piece.substr(starts[k], starts[k + 2] - starts[k]));
      return rank_of(key);
    };
    std::vector<int> ranks(n, -1);
    for (size_t k = 0; k + 1 < n; ++k) ranks[k] = pair_rank(k);
    while (starts.size() > 2) {
      int best = -1; size_t at = 0;
      for (size_t k = 0; k + 2 < starts.size(); ++k)
        if (ranks[k] >= 0 && (best < 0 || ranks[k] < best)) { best = ranks[k]; at = k; }
      if (best < 0) break;
      starts.erase(starts.begin() + at + 1);
      ranks.erase(ranks.begin() + at);
      if (at < ranks.size()) ranks[at] = pair_rank(at);
      if (at > 0) ranks[at - 1] = pair_rank(at - 1);
    }
    for (size_t k = 0; k + 1 < starts.size(); ++k) {
      key.assign(piece.substr(starts[k], starts[k + 1] - starts[k]));
      out.push_back(rank_of(key));
    }
  }

  std::unordered_map<std::string, int> table_;
};

std::vector<std::string> split_text(const std::string& text) {
  std::vector<std::pair<uint32_t, uint32_t>> pieces;
  tok::split(text, pieces);
  std::vector<std::string> out;
  out.reserve(pieces.size());
  for (auto& pc : pieces) out.push_back(text.substr(pc.first, pc.second - pc.first));
  return out;
}

// ------------------------------------------------------------------------------- packer
class BestFitPacker {
 public:
  BestFitPacker(int row_capacity, int buffer_size) : cap_(row_capacity), want_(buffer_size) {}

  void add_documents(const std::vector<std::vector<int>>& docs) {
    for (auto& d : docs) {
      if (d.empty()) continue;
      const uint64_t id = next_id_++;
      order_.insert({static_cast<int>(d.size()), id});
      docs_.emplace(id, d);
    }
  }
  bool needs_documents() const { return static_cast<int>(docs_.size()) < want_; }
  size_t size() const { return docs_.size(); }

  // Returns (num_rows, row_capacity) int64. `refill` is called (GIL held) whenever the pool is short.
  py::array_t<long long> pack(int num_rows, const py::function& refill) {
    py::array_t<long long> rows({num_rows, cap_});
    auto buf = rows.mutable_unchecked<2>();
    for (int r = 0; r < num_rows; ++r) {
      int pos = 0;
      while (pos < cap_) {
        int guard = 0;
        while (needs_documents()) {
          refill();
          if (++guard > 1000000) throw std::runtime_error("packer: refill callback does not add documents");
        }
        const int room = cap_ - pos;
        // largest length <= room, oldest among equals
        auto ub = order_.upper_bound({room, UINT64_MAX});
        if (ub != order_.begin()) {
          const int len = std::prev(ub)->first;
          auto pick = order_.lower_bound({len, 0});
          const std::vector<int>& d = docs_[pick->second];
          for (int k = 0; k < len; ++k) buf(r, pos + k) = d[k];
          pos += len;
          docs_.erase(pick->second);
          order_.erase(pick);
        } else {
          auto pick = order_.begin();   // shortest, oldest among equals: crop it to fill the row
          const std::vector<int>& d = docs_[pick->second];
          for (int k = 0; k < room; ++k) buf(r, pos + k) = d[k];
          pos = cap_;
          docs_.erase(pick->second);
          order_.erase(pick);
        }
      }
    }
    return rows;
  }

 private:
  int cap_, want_;
  uint64_t next_id_ = 0;
  std::set<std::pair<int, uint64_t>> order_;
  std::unordered_map<uint64_t, std::vector<int>> docs_;
};

}  // namespace

PYBIND11_MODULE(_tok, m) {
  m.doc() = "nanochat_b200 native tokenizer: BPE training / encoding and best-fit packing";
  m.def("train_bpe", &train_bpe, py::arg("iterator"), py::arg("vocab_size"), py::arg("threads") = 8);
  m.def("split", &split_text);
  py::class_<Encoder>(m, "Encoder")
      .def(py::init([](const std::vector<py::bytes>& tokens, const std::vector<int>& ranks) {
        std::vector<std::string> t;
        t.reserve(tokens.size());
        for (auto& b : tokens) t.push_back(static_cast<std::string>(b));
        return new Encoder(t, ranks);
      }))
      .def("encode_ordinary", &Encoder::encode_ordinary)
      .def("encode_ordinary_batch", &Encoder::encode_ordinary_batch, py::arg("texts"), py::arg("num_threads") = 8);
  py::class_<BestFitPacker>(m, "BestFitPacker")
      .def(py::init<int, int>())
      .def("add_documents", &BestFitPacker::add_documents)
      .def("needs_documents", &BestFitPacker::needs_documents)
      .def("__len__", &BestFitPacker::size)
      .def("pack", &BestFitPacker::pack);
}
