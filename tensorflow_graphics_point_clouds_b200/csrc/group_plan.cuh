// Row plan shared by the grouped projection kernels (group_plan.cu builds it).
#pragma once

#include "common.cuh"

namespace tfgpc {
namespace gp {

constexpr int kG = 4;            // samples per group
constexpr int kMaxMerge = 512;   // pairs of a group that are merged in shared memory
constexpr int kBitmapBits = 8192;  // id span of a group that is merged through a bit set
constexpr int kRowPad = 256;     // rows a kernel may read beyond the last one

struct PlanView {
  int32_t* group_begin;   // [groups + 1]
  int32_t* group_rows;    // [groups]
  int32_t* rows_id;       // [M + 3 groups + kRowPad]
  int4* rows_pair;        // [M + 3 groups + kRowPad]
  int64_t* scan_sums;
  int64_t groups;
  size_t bytes;
};

PlanView plan_view(void* buf, int64_t ns, int64_t M);

}  // namespace gp
}  // namespace tfgpc
