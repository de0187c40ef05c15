// Host-side helpers the part kinds share: matrices put together from several tensors of the weight file,
// tensor requests, rotary frequencies.
#pragma once

#include <memory>
#include <vector>

#include "device.h"
#include "json.h"
#include "weights.h"

namespace sandy {
namespace part_helpers {

std::shared_ptr<float> alloc_f32(size_t n);
HostTensor host_f32(std::shared_ptr<float> data, std::vector<int64_t> shape);
// Rows of several [n_i, cols] matrices one under the other.
HostTensor stack_rows(const std::vector<const HostTensor*>& parts, int64_t cols);
// Columns of several [rows, n_i] matrices side by side; with `group` > 0 every group of `group` columns is widened
// to `group_padded` with zero columns.
struct ColumnPart { const HostTensor* t; int64_t cols; int64_t group; int64_t group_padded; };
HostTensor join_columns(const std::vector<ColumnPart>& parts, int64_t rows, int64_t total_cols);
TensorRequest want(std::vector<int64_t> shape, const char* init = "weight");
int64_t round_up(int64_t n, int64_t m);
// f_i = base^(-2i / dims), i < dims / 2, with an optional long-context rescaling {factor, low, high, original}.
std::vector<float> rotary_frequencies(int dims, double base, const Json* scaling);
DeviceWeight floats_to_device(const std::vector<float>& v);

}  // namespace part_helpers
}  // namespace sandy
