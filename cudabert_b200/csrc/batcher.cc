// Length-bucketing batcher of the file-to-file engine, as native host code.  It restates what
// the reference's reader stage does in Python (engine.py:12-130: `batch_container`,
// `queue_manager.put / enqueue / force_enqueue`; utils.py:3-13: `optimize_batch`; utils.py:49-56:
// the valid length of a line): tokenised lines are sorted into buckets by valid length
// (boundaries b[0] < b[1] < ... ; bucket q takes lengths in (b[q], b[q+1]], the last bucket
// everything longer), a bucket that holds `batch_size` lines becomes a ready batch, ready batches
// leave in the order of their first line number (which keeps the writer's re-ordering window
// short), and every batch is right-trimmed to its own longest line.  A flush turns the partly
// filled buckets into batches (end of input, or the writer asking for its missing lines).
//
// The three int32 arrays a batch pops into are exactly the [rows, seq] ids / segment ids / mask
// the forward pass takes; the kernels then pack away what padding is left inside the batch.
#include "../../include/cudabert.h"

#include <algorithm>
#include <climits>
#include <cstring>
#include <deque>
#include <memory>
#include <vector>

namespace {

struct Line {
  long long index;
  int length;          // valid length: 1 + position of the last mask entry equal to 1
  std::vector<int> row;  // ids | seg | mask, each `stored` long (the row as it was put)
  int stored;
};

struct Batch {
  std::vector<Line> lines;
  int seq;  // longest valid length in the batch
};

struct Bucket {
  std::vector<Line> filling;
  std::deque<Batch> ready;
};

struct Batcher {
  std::vector<int> bounds;
  std::vector<Bucket> buckets;
  int batch_size;
  int max_seq;
  long long lines_in = 0, lines_out = 0;

  void close(Bucket& b) {
    if (b.filling.empty()) return;
    Batch batch;
    batch.seq = 0;
    for (const Line& l : b.filling) batch.seq = std::max(batch.seq, l.length);
    batch.lines.swap(b.filling);
    b.ready.push_back(std::move(batch));
  }
  // the bucket whose oldest ready batch starts at the smallest line number; nullptr if none is ready
  Bucket* next() {
    Bucket* best = nullptr;
    long long best_index = LLONG_MAX;
    for (Bucket& b : buckets)
      if (!b.ready.empty() && b.ready.front().lines.front().index < best_index) {
        best = &b;
        best_index = b.ready.front().lines.front().index;
      }
    return best;
  }
  int ready_count() const {
    size_t n = 0;
    for (const Bucket& b : buckets) n += b.ready.size();
    return static_cast<int>(n);
  }
};

}  // namespace

extern "C" {

void* cudabert_batcher_create(const int* boundaries, int n_boundaries, int batch_size, int max_seq_length) {
  if (!boundaries || n_boundaries < 2 || batch_size < 1 || max_seq_length < 1) return nullptr;
  for (int i = 1; i < n_boundaries; ++i)
    if (boundaries[i] < boundaries[i - 1]) return nullptr;
  std::unique_ptr<Batcher> b(new Batcher);
  b->bounds.assign(boundaries, boundaries + n_boundaries);
  b->buckets.resize(n_boundaries - 1);
  b->batch_size = batch_size;
  b->max_seq = max_seq_length;
  return b.release();
}

void cudabert_batcher_destroy(void* batcher) { delete static_cast<Batcher*>(batcher); }

int cudabert_batcher_put(void* batcher, long long line_index, const int* ids, const int* seg, const int* mask, int n) {
  Batcher* b = static_cast<Batcher*>(batcher);
  if (!b || !ids || !seg || !mask || n < 1 || n > b->max_seq) return -1;
  int length = n;  // a mask without a 1 keeps the whole row, like a line the reference cannot measure
  for (int i = n - 1; i >= 0; --i)
    if (mask[i] == 1) { length = i + 1; break; }
  Line l;
  l.index = line_index;
  l.length = length;
  // the whole row is kept: a batch is trimmed to its LONGEST line, and a shorter line then shows
  // its own entries beyond its valid length, as a slice of the reference's padded row does
  l.stored = n;
  l.row.resize(static_cast<size_t>(3) * n);
  std::memcpy(l.row.data(), ids, sizeof(int) * n);
  std::memcpy(l.row.data() + n, seg, sizeof(int) * n);
  std::memcpy(l.row.data() + 2 * static_cast<size_t>(n), mask, sizeof(int) * n);
  size_t q = 0;
  while (q + 1 < b->buckets.size() && length > b->bounds[q + 1]) ++q;
  Bucket& bucket = b->buckets[q];
  bucket.filling.push_back(std::move(l));
  ++b->lines_in;
  if (static_cast<int>(bucket.filling.size()) == b->batch_size) b->close(bucket);
  return length;
}

int cudabert_batcher_flush(void* batcher) {
  Batcher* b = static_cast<Batcher*>(batcher);
  if (!b) return -1;
  for (Bucket& bucket : b->buckets) b->close(bucket);
  return b->ready_count();
}

int cudabert_batcher_ready(void* batcher) {
  Batcher* b = static_cast<Batcher*>(batcher);
  return b ? b->ready_count() : -1;
}

long long cudabert_batcher_pending(void* batcher) {
  Batcher* b = static_cast<Batcher*>(batcher);
  return b ? b->lines_in - b->lines_out : -1;
}

int cudabert_batcher_next(void* batcher, int* rows, int* seq, long long* first_line) {
  Batcher* b = static_cast<Batcher*>(batcher);
  if (!b) return -1;
  Bucket* bucket = b->next();
  if (!bucket) return 0;
  const Batch& batch = bucket->ready.front();
  if (rows) *rows = static_cast<int>(batch.lines.size());
  if (seq) *seq = batch.seq;
  if (first_line) *first_line = batch.lines.front().index;
  return 1;
}

int cudabert_batcher_pop(void* batcher, long long* line_index, int* ids, int* seg, int* mask) {
  Batcher* b = static_cast<Batcher*>(batcher);
  if (!b || !line_index || !ids || !seg || !mask) return -1;
  Bucket* bucket = b->next();
  if (!bucket) return 0;
  Batch batch = std::move(bucket->ready.front());
  bucket->ready.pop_front();
  const int rows = static_cast<int>(batch.lines.size()), seq = batch.seq;
  for (int r = 0; r < rows; ++r) {
    const Line& l = batch.lines[r];
    line_index[r] = l.index;
    int* dst[3] = {ids + static_cast<size_t>(r) * seq, seg + static_cast<size_t>(r) * seq,
                   mask + static_cast<size_t>(r) * seq};
    const int take = std::min(seq, l.stored);
    for (int a = 0; a < 3; ++a) {
      std::memcpy(dst[a], l.row.data() + static_cast<size_t>(a) * l.stored, sizeof(int) * take);
      std::fill(dst[a] + take, dst[a] + seq, 0);  // a row shorter than the batch: id 0, segment 0, mask 0
    }
  }
  b->lines_out += rows;
  return rows;
}

}  // extern "C"
