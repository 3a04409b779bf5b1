// The engine's reader stage as native host code: several threads read lines of the input file,
// tokenise them (tokenizer.cc) and drop them into the length buckets (batcher.cc); the caller pulls
// finished batches together with the raw text of their lines, which the writer stage needs.
// It does what the reference's reader process does one line at a time in Python
// (engine.py:266-280 `_engine_preprocess`, with apps/tokenlizer.py:136-147 as the per-line function):
//   line number = position in the file (after an optional header line);
//   text_a, text_b = the line without NUL bytes and trailing whitespace, split at tabs;
//   raw text kept for the writer = the same fields joined by tabs again.
// Lines reach the buckets in slightly shuffled order (whichever thread finishes first), which changes
// nothing downstream: batches still leave by smallest first line number and the writer restores
// the input order.  Lines end as in Python's text mode (universal newlines): at "\n", at "\r\n" and at
// a lone "\r", so both readers number the lines of any file alike.  A line the tokenizer or the
// buckets refuse is counted and stops the stream (cudabert_reader_next returns -1) instead of
// leaving a hole in the line numbers that the writer would only notice at the end.
#include "../../include/cudabert.h"

#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

// trailing characters str.rstrip() removes, as UTF-8: ASCII white space, U+0085, U+00A0, U+1680,
// U+2000..U+200A, U+2028, U+2029, U+202F, U+205F, U+3000
size_t rstrip_len(const std::string& s) {
  size_t n = s.size();
  for (;;) {
    if (n == 0) return 0;
    const unsigned char c = static_cast<unsigned char>(s[n - 1]);
    if (c == ' ' || (c >= 9 && c <= 13) || (c >= 28 && c <= 31)) { --n; continue; }
    if (n >= 2) {
      const unsigned char b = static_cast<unsigned char>(s[n - 2]);
      if (b == 0xC2 && (c == 0x85 || c == 0xA0)) { n -= 2; continue; }
    }
    if (n >= 3) {
      const unsigned char a = static_cast<unsigned char>(s[n - 3]), b = static_cast<unsigned char>(s[n - 2]);
      const bool sp = (a == 0xE1 && b == 0x9A && c == 0x80) ||                                  // U+1680
                      (a == 0xE2 && b == 0x80 && (c <= 0x8A || c == 0xA8 || c == 0xA9 || c == 0xAF)) ||  // U+2000-200A, 2028, 2029, 202F
                      (a == 0xE2 && b == 0x81 && c == 0x9F) ||                                  // U+205F
                      (a == 0xE3 && b == 0x80 && c == 0x80);                                    // U+3000
      if (sp && (a != 0xE2 || b != 0x80 || c >= 0x80)) { n -= 3; continue; }
    }
    return n;
  }
}

struct Reader {
  std::FILE* file = nullptr;
  void* tokenizer = nullptr;  // not owned
  void* batcher = nullptr;    // owned
  int max_seq = 0;
  size_t max_ready = 64;      // back-pressure: batches the threads may run ahead of the consumer

  std::mutex file_mu;
  long long next_index = 0;

  std::mutex mu;  // batcher, raw, counters
  std::condition_variable batch_ready, room;
  std::map<long long, std::string> raw;  // raw text of the lines inside the batcher
  std::string last_raw;                  // raw text of the batch taken last, line after line
  // the batch cudabert_reader_next took out of the buckets, until cudabert_reader_pop copies it
  std::vector<long long> cur_index, cur_offsets;
  std::vector<int> cur_ids, cur_seg, cur_mask;
  int cur_seq = 0;
  int threads_running = 0;
  bool stop = false;
  long long lines_read = 0;
  long long rejected = 0, first_rejected = -1;

  // Next line of the file without its terminator ("\n", "\r\n" or a lone "\r") and without NUL
  // bytes; false at the end of the file.  Called under file_mu.
  bool read_line(std::string& line) {
    line.clear();
    int c = getc_unlocked(file);
    if (c == EOF) return false;
    for (; c != EOF; c = getc_unlocked(file)) {
      if (c == '\n') break;
      if (c == '\r') {
        const int next = getc_unlocked(file);
        if (next != '\n' && next != EOF) ungetc(next, file);
        break;
      }
      if (c != '\0') line.push_back(static_cast<char>(c));
    }
    return true;
  }

  std::vector<std::thread> threads;

  void work() {
    std::vector<int> ids(max_seq), mask(max_seq), seg(max_seq);
    std::string line;
    for (;;) {
      long long index;
      {
        std::lock_guard<std::mutex> lk(file_mu);
        if (!read_line(line)) break;
        index = next_index++;
      }
      line.resize(rstrip_len(line));
      const size_t tab = line.find('\t');
      std::string a = line.substr(0, tab), b;
      if (tab != std::string::npos) {
        const size_t tab2 = line.find('\t', tab + 1);
        b = line.substr(tab + 1, tab2 == std::string::npos ? std::string::npos : tab2 - tab - 1);
      }
      const int n_tok = cudabert_tokenizer_encode_pair(tokenizer, a.c_str(), b.empty() ? nullptr : b.c_str(), max_seq,
                                                       ids.data(), mask.data(), seg.data());
      std::unique_lock<std::mutex> lk(mu);
      room.wait(lk, [&] { return stop || static_cast<size_t>(cudabert_batcher_ready(batcher)) < max_ready; });
      if (stop) break;
      if (n_tok >= 0 && cudabert_batcher_put(batcher, index, ids.data(), seg.data(), mask.data(), max_seq) >= 0) {
        raw[index] = line;
        ++lines_read;
      } else {
        if (rejected++ == 0) first_rejected = index;
        batch_ready.notify_all();
      }
      if (cudabert_batcher_ready(batcher) > 0) batch_ready.notify_all();
    }
    std::lock_guard<std::mutex> lk(mu);
    if (--threads_running == 0) {
      cudabert_batcher_flush(batcher);  // end of input: the partly filled buckets leave too
      batch_ready.notify_all();
    }
  }
};

}  // namespace

extern "C" {

void* cudabert_reader_create(const char* input_path, void* tokenizer, int max_seq_length, const int* boundaries,
                             int n_boundaries, int batch_size, int threads, long long skip_lines,
                             long long first_index) {
  if (!input_path || !tokenizer || max_seq_length < 3 || threads < 1 || threads > 256 || skip_lines < 0) return nullptr;
  std::unique_ptr<Reader> r(new Reader);
  r->batcher = cudabert_batcher_create(boundaries, n_boundaries, batch_size, max_seq_length);
  if (!r->batcher) return nullptr;
  r->file = std::fopen(input_path, "rb");
  if (!r->file) {
    cudabert_batcher_destroy(r->batcher);
    return nullptr;
  }
  {
    std::string skipped;
    for (long long i = 0; i < skip_lines; ++i)
      if (!r->read_line(skipped)) break;  // fewer lines than asked: nothing left to read
  }
  r->next_index = first_index;
  r->tokenizer = tokenizer;
  r->max_seq = max_seq_length;
  r->threads_running = threads;
  Reader* raw_ptr = r.get();
  for (int i = 0; i < threads; ++i) r->threads.emplace_back([raw_ptr] { raw_ptr->work(); });
  return r.release();
}

void cudabert_reader_destroy(void* reader) {
  Reader* r = static_cast<Reader*>(reader);
  if (!r) return;
  {
    std::lock_guard<std::mutex> lk(r->mu);
    r->stop = true;
  }
  r->room.notify_all();
  for (std::thread& t : r->threads) t.join();
  std::fclose(r->file);
  cudabert_batcher_destroy(r->batcher);
  delete r;
}

int cudabert_reader_next(void* reader, int* rows, int* seq, long long* first_line) {
  Reader* r = static_cast<Reader*>(reader);
  if (!r) return -1;
  std::unique_lock<std::mutex> lk(r->mu);
  r->batch_ready.wait(lk, [&] {
    return cudabert_batcher_ready(r->batcher) > 0 || r->threads_running == 0 || r->rejected > 0;
  });
  if (r->rejected > 0) return -1;  // a line was refused: its number would be missing downstream
  int n_rows = 0, n_seq = 0;
  long long first = 0;
  if (cudabert_batcher_next(r->batcher, &n_rows, &n_seq, &first) != 1) return 0;  // every thread is done and nothing is left
  // The batch is taken out of the buckets here, under the lock, and parked: the threads keep
  // filling the buckets, and a batch with a smaller first line may be ready by the time the caller
  // has sized its arrays.
  r->cur_index.resize(n_rows);
  r->cur_ids.resize(static_cast<size_t>(n_rows) * n_seq);
  r->cur_seg.resize(r->cur_ids.size());
  r->cur_mask.resize(r->cur_ids.size());
  const int got = cudabert_batcher_pop(r->batcher, r->cur_index.data(), r->cur_ids.data(), r->cur_seg.data(),
                                       r->cur_mask.data());
  if (got != n_rows) return -1;
  r->cur_seq = n_seq;
  r->cur_offsets.resize(n_rows + 1);
  r->last_raw.clear();
  for (int i = 0; i < n_rows; ++i) {
    r->cur_offsets[i] = static_cast<long long>(r->last_raw.size());
    auto it = r->raw.find(r->cur_index[i]);
    if (it != r->raw.end()) {
      r->last_raw += it->second;
      r->raw.erase(it);
    }
  }
  r->cur_offsets[n_rows] = static_cast<long long>(r->last_raw.size());
  r->room.notify_all();
  if (rows) *rows = n_rows;
  if (seq) *seq = n_seq;
  if (first_line) *first_line = first;
  return 1;
}

int cudabert_reader_pop(void* reader, long long* line_index, int* ids, int* seg, int* mask, long long* raw_offsets) {
  Reader* r = static_cast<Reader*>(reader);
  if (!r || !line_index || !ids || !seg || !mask || !raw_offsets) return -1;
  std::lock_guard<std::mutex> lk(r->mu);
  const int rows = static_cast<int>(r->cur_index.size());
  if (rows == 0) return 0;
  std::memcpy(line_index, r->cur_index.data(), sizeof(long long) * rows);
  std::memcpy(ids, r->cur_ids.data(), sizeof(int) * r->cur_ids.size());
  std::memcpy(seg, r->cur_seg.data(), sizeof(int) * r->cur_seg.size());
  std::memcpy(mask, r->cur_mask.data(), sizeof(int) * r->cur_mask.size());
  std::memcpy(raw_offsets, r->cur_offsets.data(), sizeof(long long) * (rows + 1));
  r->cur_index.clear();
  return rows;
}

long long cudabert_reader_raw(void* reader, char* buf, long long capacity) {
  Reader* r = static_cast<Reader*>(reader);
  if (!r || (capacity > 0 && !buf)) return -1;
  std::lock_guard<std::mutex> lk(r->mu);
  const long long n = static_cast<long long>(r->last_raw.size());
  if (capacity > 0) std::memcpy(buf, r->last_raw.data(), static_cast<size_t>(n < capacity ? n : capacity));
  return n;
}

int cudabert_reader_flush(void* reader) {
  Reader* r = static_cast<Reader*>(reader);
  if (!r) return -1;
  std::lock_guard<std::mutex> lk(r->mu);
  const int n = cudabert_batcher_flush(r->batcher);
  if (n > 0) r->batch_ready.notify_all();
  return n;
}

long long cudabert_reader_rejected(void* reader, long long* first_index) {
  Reader* r = static_cast<Reader*>(reader);
  if (!r) return -1;
  std::lock_guard<std::mutex> lk(r->mu);
  if (first_index) *first_index = r->first_rejected;
  return r->rejected;
}

long long cudabert_reader_lines(void* reader) {
  Reader* r = static_cast<Reader*>(reader);
  if (!r) return -1;
  std::lock_guard<std::mutex> lk(r->mu);
  return r->lines_read;
}

}  // extern "C"
