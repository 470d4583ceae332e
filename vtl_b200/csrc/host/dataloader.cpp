// datasets.DataLoader (datasets/dataloader.v) over a dataset that lives on the device: the same
// index bookkeeping (sequential or Fisher-Yates order from the reference's LCG, :168-177 and
// :316-331; drop_last; len; reset per epoch; split), with the rows of a batch gathered by one
// kernel (vtlb_gather_rows_f32) instead of element-by-element host loops (:41-143).
#include <cstring>

#include "vtl_host.hpp"

namespace vtl {

namespace {
// LcgRng (dataloader.v:316-331)
struct LcgRng {
  uint64_t state;
  explicit LcgRng(uint64_t seed) : state(seed == 0 ? 1 : seed) {}
  uint64_t next() {
    state = state * 6364136223846793005ull + 1442695040888963407ull;
    return state;
  }
};
}  // namespace

DataLoader::DataLoader(const Tensor& dataset_, const Tensor& labels_, DataLoaderConfig c)
    : dataset(dataset_), labels(labels_), batch_size(c.batch_size), shuffle(c.shuffle), drop_last(c.drop_last),
      seed(c.seed) {
  if (!dataset.defined() || dataset.shape().empty()) throw Error(VTLB_EINVAL, "DataLoader: dataset must have a batch dimension");
  if (batch_size <= 0) throw Error(VTLB_EINVAL, "DataLoader: batch_size must be positive");
  const int n = dataset.shape()[0];
  if (labels.defined() && (labels.shape().empty() || labels.shape()[0] != n))
    throw Error(VTLB_EINVAL, "DataLoader: dataset and labels differ in their first dimension");
  indices.resize(n);
  for (int i = 0; i < n; ++i) indices[i] = i;
  if (shuffle) shuffle_indices();
  indices_dirty_ = true;
}

// dataloader.v:168-177: Fisher-Yates from the back with rng.next() % (i + 1), seed + epoch
void DataLoader::shuffle_indices() {
  LcgRng rng(seed + (uint64_t)epoch);
  for (int i = (int)indices.size() - 1; i > 0; --i) {
    const int j = (int)(rng.next() % (uint64_t)(i + 1));
    std::swap(indices[i], indices[j]);
  }
  indices_dirty_ = true;
}

void DataLoader::reset() {  // :160-165
  ++epoch;
  if (shuffle) shuffle_indices();
}

int DataLoader::len() const {  // :146-154
  if (indices.empty()) return 0;
  if (drop_last) return (int)indices.size() / batch_size;
  return ((int)indices.size() + batch_size - 1) / batch_size;
}

bool DataLoader::range(int i, int& start, int& end) const {  // :46-63
  if (indices.empty() || i < 0) return false;
  start = i * batch_size;
  if (start >= (int)indices.size()) return false;
  end = start + batch_size;
  if (end > (int)indices.size()) {
    if (drop_last) return false;
    end = (int)indices.size();
  }
  return true;
}

void DataLoader::sync_indices() {
  if (!indices_dirty_) return;
  Session* s = dataset.session();
  if (!d_indices_ || d_indices_->bytes < indices.size() * sizeof(int))
    d_indices_ = std::make_shared<DeviceBuf>(s, std::max<size_t>(indices.size() * sizeof(int), 16));
  s->check(vtlb_h2d(s->ctx, d_indices_->ptr, indices.data(), indices.size() * sizeof(int)));
  s->sync();  // `indices` may change as soon as we return
  indices_dirty_ = false;
}

Tensor DataLoader::gather(const Tensor& src, int start, int end) {
  Session* s = src.session();
  std::vector<int> shape = src.shape();
  const size_t row = src.size() / (size_t)shape[0];
  const int rows = shape[0];
  shape[0] = end - start;
  Tensor out = Tensor::empty(s, shape);
  s->check(vtlb_gather_rows_f32(s->ctx, src.data(), rows, row, static_cast<const int*>(d_indices_->ptr) + start,
                                end - start, out.data(), 0));
  return out;
}

bool DataLoader::batch(int i, Tensor* features) {
  int start, end;
  if (!range(i, start, end)) return false;
  sync_indices();
  *features = gather(dataset, start, end);
  return true;
}

bool DataLoader::batch_with_labels(int i, Tensor* features, Tensor* labels_out) {
  if (!labels.defined()) return false;  // :91-93
  int start, end;
  if (!range(i, start, end)) return false;
  sync_indices();
  *features = gather(dataset, start, end);
  *labels_out = gather(labels, start, end);
  return true;
}

// :270-306: the last val_fraction of the current order becomes the validation loader
std::pair<std::unique_ptr<DataLoader>, std::unique_ptr<DataLoader>> DataLoader::split(double val_fraction) const {
  const int n = (int)indices.size();
  const int val_size = (int)((double)n * val_fraction);
  const int train_size = n - val_size;
  DataLoaderConfig c;
  c.batch_size = batch_size;
  c.shuffle = false;
  c.drop_last = drop_last;
  c.seed = seed;
  auto train = std::unique_ptr<DataLoader>(new DataLoader(dataset, labels, c));
  train->indices.assign(indices.begin(), indices.begin() + train_size);
  train->epoch = epoch;
  train->indices_dirty_ = true;
  c.drop_last = false;
  auto val = std::unique_ptr<DataLoader>(new DataLoader(dataset, labels, c));
  val->indices.assign(indices.begin() + train_size, indices.end());
  val->epoch = 0;
  val->indices_dirty_ = true;
  return {std::move(train), std::move(val)};
}

}  // namespace vtl
