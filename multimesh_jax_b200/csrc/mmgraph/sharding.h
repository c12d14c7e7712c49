// Sharded-array descriptors and the sharding algebra of the MPMD compiler:
// device ranges, tiled shardings over a submesh, logical->physical mapping,
// resize across unequal submeshes, mesh equivalence and reshard planning.
//
// Information content follows the reference's ShardedShape
// (src/pjrt_client/mm_sharding.cc:275-432, 583-671): dtype, global size per
// dimension, how each dimension is split over mesh axes, and the contiguous
// device range that owns the array. Devices outside the range hold nothing;
// every device in the range holds exactly one contiguous row-major tile.
#pragma once
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "json.h"

namespace mmg {

enum class DType : int {
  F32, F16, BF16, F64, I8, I16, I32, I64, U8, U16, U32, U64, BOOL, F8E4M3, F8E5M2, kCount
};
size_t DTypeSize(DType t);
const char* DTypeName(DType t);
DType DTypeFromName(const std::string& name);

// Contiguous range of global device ids [start, start + n).
struct DeviceRange {
  int start = 0;
  int n = 0;
  static DeviceRange Create(int start, int n) { return DeviceRange{start, n}; }
  // Builds a range from an ascending contiguous list; throws otherwise.
  static DeviceRange FromList(const std::vector<int>& devices);
  int stop() const { return start + n; }
  int size() const { return n; }
  bool Contains(int device) const { return device >= start && device < start + n; }
  bool Contains(const DeviceRange& o) const { return o.start >= start && o.stop() <= stop(); }
  int operator[](int i) const { return start + i; }
  bool operator==(const DeviceRange& o) const { return start == o.start && n == o.n; }
  bool operator!=(const DeviceRange& o) const { return !(*this == o); }
  bool operator<(const DeviceRange& o) const { return start != o.start ? start < o.start : n < o.n; }
  std::vector<int> ToList() const;
  std::string ToString() const;
};

// One half-open box of element indices per dimension.
struct Box {
  std::vector<int64_t> lo, hi;
  int64_t Volume() const;
  bool Empty() const;
  static Box Intersect(const Box& a, const Box& b);
  bool operator==(const Box& o) const { return lo == o.lo && hi == o.hi; }
};

// A tiled sharding of a tensor over a mesh laid out row-major on `devices`.
// dim_axes[d] lists the mesh axes (major to minor) that split tensor dim d.
// Mesh axes used by no dimension replicate the tile.
struct ShardedShape {
  DType dtype = DType::F32;
  std::vector<int64_t> sizes;
  std::vector<std::vector<int>> dim_axes;
  std::vector<int> mesh_dims;
  DeviceRange devices;

  static ShardedShape Replicated(DType dtype, std::vector<int64_t> sizes, DeviceRange devices);
  int rank() const { return static_cast<int>(sizes.size()); }
  bool IsScalar() const { return sizes.empty(); }
  int Shards(int dim) const;
  int TotalShards() const;
  int Replication() const { return devices.n / std::max(1, TotalShards()); }
  bool IsReplicated() const { return TotalShards() == 1; }
  // Local tile shape (same on every device; sizes divide evenly).
  std::vector<int64_t> ShardSize() const;
  int64_t ShardElements() const;
  int64_t ShardBytes() const { return ShardElements() * static_cast<int64_t>(DTypeSize(dtype)); }
  int64_t GlobalElements() const;
  // Shard index along `dim` held by the i-th device of the range.
  int ShardIndex(int device_ordinal, int dim) const;
  // Element box held by the i-th device of the range.
  Box TileBox(int device_ordinal) const;
  // {size, shard count, position of the first mesh axis} per dimension.
  struct Dim { int64_t size; int shards; int permutation; };
  std::vector<Dim> CanonicalDims() const;
  bool Valid(std::string* why = nullptr) const;
  std::string Key() const;  // stable text form, usable as a pool / dedup key
  Json ToJson() const;
  static ShardedShape FromJson(const Json& j);
  bool operator==(const ShardedShape& o) const { return Key() == o.Key(); }
};

// Same tiles on the same devices (dtype and sizes equal, every device holds
// the same box), regardless of how the mesh axes are named or factored.
bool MeshEquivalent(const ShardedShape& a, const ShardedShape& b);

// A reshard between producer layout `src` and consumer layout `dst` is not
// needed iff both are replicated and src devices contain dst devices, or the
// device ranges and tiles agree (src/pjrt_client/mpmd_insert_reshard.cc:33-43).
bool NeedsReshard(const ShardedShape& src, const ShardedShape& dst);

// Re-expresses `s` on a submesh with `dst_devices` devices: when the mesh is
// one-dimensional in effect (identity permutation) the first sharded dimension
// is rescaled by dst/src if that divides evenly and fits; otherwise the result
// is replicated and *ok is false (src/pjrt_client/mm_sharding.cc:98-162).
ShardedShape ResizeSharding(const ShardedShape& s, DeviceRange dst_devices, bool* ok);

// Replaces the sharding of the listed dims by replication.
ShardedShape ReplicateDims(const ShardedShape& s, const std::vector<int>& dims);

// Logical -> physical: walks `logical_axes` (priority order of (logical name,
// mesh axis name)); a mesh axis is given to a tensor dim whose name set
// contains the logical name if the axis is still unused on this tensor and
// shards_so_far * |axis| <= dim size (and divides it)
// (src/pjrt_client/mpmd_logical_to_gspmd_sharding.cc:38-83).
ShardedShape LogicalToPhysical(DType dtype, const std::vector<int64_t>& sizes,
                               const std::vector<std::vector<std::string>>& axes,
                               const std::vector<std::pair<std::string, std::string>>& logical_axes,
                               const std::vector<std::string>& mesh_axis_names,
                               const std::vector<int>& mesh_dims, DeviceRange devices);

// One rectangular copy of a reshard: elements `box` (global coordinates) move
// from src device ordinal (global id src_device) to dst_device.
struct ReshardChunk {
  int src_device;
  int dst_device;
  Box box;
  std::vector<int64_t> src_offset;  // box.lo relative to the source tile
  std::vector<int64_t> dst_offset;  // box.lo relative to the destination tile
};
struct ReshardPlan {
  ShardedShape src, dst;
  std::vector<ReshardChunk> chunks;  // grouped by dst_device, ascending
  int64_t BytesOverLinks() const;    // bytes whose src and dst devices differ
  int64_t BytesTotal() const;
};
// Every destination tile is covered exactly once; among source replicas that
// hold a needed box the destination device itself is preferred, then replicas
// are spread round-robin so that no single source serves every destination.
ReshardPlan PlanReshard(const ShardedShape& src, const ShardedShape& dst);

}  // namespace mmg
