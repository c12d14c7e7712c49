#include "sharding.h"

#include <algorithm>
#include <map>
#include <sstream>
#include <stdexcept>

namespace mmg {

static const struct { DType t; const char* name; size_t size; } kDTypes[] = {
    {DType::F32, "float32", 4},   {DType::F16, "float16", 2},   {DType::BF16, "bfloat16", 2},
    {DType::F64, "float64", 8},   {DType::I8, "int8", 1},       {DType::I16, "int16", 2},
    {DType::I32, "int32", 4},     {DType::I64, "int64", 8},     {DType::U8, "uint8", 1},
    {DType::U16, "uint16", 2},    {DType::U32, "uint32", 4},    {DType::U64, "uint64", 8},
    {DType::BOOL, "bool", 1},     {DType::F8E4M3, "float8_e4m3fn", 1}, {DType::F8E5M2, "float8_e5m2", 1},
};

size_t DTypeSize(DType t) {
  for (auto& d : kDTypes) if (d.t == t) return d.size;
  return 4;
}
const char* DTypeName(DType t) {
  for (auto& d : kDTypes) if (d.t == t) return d.name;
  return "float32";
}
DType DTypeFromName(const std::string& name) {
  std::string n = name;
  if (n.rfind("torch.", 0) == 0) n = n.substr(6);
  for (auto& d : kDTypes) if (n == d.name) return d.t;
  throw std::runtime_error("unsupported dtype " + name);
}

DeviceRange DeviceRange::FromList(const std::vector<int>& devices) {
  if (devices.empty()) return DeviceRange{0, 0};
  for (size_t i = 1; i < devices.size(); ++i)
    if (devices[i] != devices[i - 1] + 1)
      throw std::runtime_error("device lists must be contiguous ascending ranges");
  return DeviceRange{devices[0], static_cast<int>(devices.size())};
}
std::vector<int> DeviceRange::ToList() const {
  std::vector<int> v(n);
  for (int i = 0; i < n; ++i) v[i] = start + i;
  return v;
}
std::string DeviceRange::ToString() const {
  std::ostringstream os;
  os << "[" << start << "," << stop() << ")";
  return os.str();
}

int64_t Box::Volume() const {
  int64_t v = 1;
  for (size_t i = 0; i < lo.size(); ++i) v *= std::max<int64_t>(0, hi[i] - lo[i]);
  return v;
}
bool Box::Empty() const {
  for (size_t i = 0; i < lo.size(); ++i) if (hi[i] <= lo[i]) return true;
  return false;
}
Box Box::Intersect(const Box& a, const Box& b) {
  Box r;
  r.lo.resize(a.lo.size());
  r.hi.resize(a.lo.size());
  for (size_t i = 0; i < a.lo.size(); ++i) {
    r.lo[i] = std::max(a.lo[i], b.lo[i]);
    r.hi[i] = std::min(a.hi[i], b.hi[i]);
  }
  return r;
}

ShardedShape ShardedShape::Replicated(DType dtype, std::vector<int64_t> sizes, DeviceRange devices) {
  ShardedShape s;
  s.dtype = dtype;
  s.dim_axes.assign(sizes.size(), {});
  s.sizes = std::move(sizes);
  s.mesh_dims = {devices.n};
  s.devices = devices;
  return s;
}
int ShardedShape::Shards(int dim) const {
  int n = 1;
  for (int a : dim_axes[dim]) n *= mesh_dims[a];
  return n;
}
int ShardedShape::TotalShards() const {
  int n = 1;
  for (int d = 0; d < rank(); ++d) n *= Shards(d);
  return n;
}
std::vector<int64_t> ShardedShape::ShardSize() const {
  std::vector<int64_t> out(sizes.size());
  for (int d = 0; d < rank(); ++d) out[d] = sizes[d] / Shards(d);
  return out;
}
int64_t ShardedShape::ShardElements() const {
  int64_t n = 1;
  for (int64_t s : ShardSize()) n *= s;
  return n;
}
int64_t ShardedShape::GlobalElements() const {
  int64_t n = 1;
  for (int64_t s : sizes) n *= s;
  return n;
}
int ShardedShape::ShardIndex(int ordinal, int dim) const {
  // mesh coordinates of the device, row-major over mesh_dims
  int idx = 0;
  for (int a : dim_axes[dim]) {
    int stride = 1;
    for (size_t k = a + 1; k < mesh_dims.size(); ++k) stride *= mesh_dims[k];
    const int coord = (ordinal / stride) % mesh_dims[a];
    idx = idx * mesh_dims[a] + coord;
  }
  return idx;
}
Box ShardedShape::TileBox(int ordinal) const {
  Box b;
  b.lo.resize(rank());
  b.hi.resize(rank());
  for (int d = 0; d < rank(); ++d) {
    const int64_t per = sizes[d] / Shards(d);
    const int i = ShardIndex(ordinal, d);
    b.lo[d] = i * per;
    b.hi[d] = (i + 1) * per;
  }
  return b;
}
std::vector<ShardedShape::Dim> ShardedShape::CanonicalDims() const {
  std::vector<Dim> out;
  for (int d = 0; d < rank(); ++d)
    out.push_back(Dim{sizes[d], Shards(d), dim_axes[d].empty() ? -1 : dim_axes[d][0]});
  return out;
}
bool ShardedShape::Valid(std::string* why) const {
  auto fail = [&](const std::string& m) { if (why) *why = m; return false; };
  int mesh = 1;
  for (int m : mesh_dims) mesh *= m;
  if (mesh != devices.n) return fail("mesh size does not match device count");
  if (dim_axes.size() != sizes.size()) return fail("dim_axes rank mismatch");
  std::vector<int> used(mesh_dims.size(), 0);
  for (int d = 0; d < rank(); ++d) {
    for (int a : dim_axes[d]) {
      if (a < 0 || a >= static_cast<int>(mesh_dims.size())) return fail("mesh axis out of range");
      if (used[a]++) return fail("mesh axis used twice");
    }
    if (sizes[d] % Shards(d)) return fail("dimension not evenly divisible by its shard count");
  }
  return true;
}
std::string ShardedShape::Key() const {
  std::ostringstream os;
  os << DTypeName(dtype) << "[";
  for (int d = 0; d < rank(); ++d) {
    if (d) os << ",";
    os << sizes[d];
    if (!dim_axes[d].empty()) {
      os << "/";
      for (size_t i = 0; i < dim_axes[d].size(); ++i) os << (i ? "." : "") << dim_axes[d][i];
    }
  }
  os << "]m(";
  for (size_t i = 0; i < mesh_dims.size(); ++i) os << (i ? "," : "") << mesh_dims[i];
  os << ")@" << devices.ToString();
  return os.str();
}
Json ShardedShape::ToJson() const {
  Json j = Json::object();
  j.set("dtype", Json::string(DTypeName(dtype)));
  Json dims = Json::array();
  auto canon = CanonicalDims();
  for (int d = 0; d < rank(); ++d) {
    Json e = Json::object();
    e.set("size", Json::number(static_cast<double>(sizes[d])));
    e.set("sharding", Json::number(canon[d].shards));
    e.set("permutation", Json::number(canon[d].permutation));
    Json ax = Json::array();
    for (int a : dim_axes[d]) ax.push(Json::number(a));
    e.set("mesh_axes", ax);
    dims.push(e);
  }
  j.set("dims", dims);
  Json mesh = Json::array();
  for (int m : mesh_dims) mesh.push(Json::number(m));
  j.set("mesh_dims", mesh);
  Json dev = Json::object();
  dev.set("start", Json::number(devices.start));
  dev.set("num_devices", Json::number(devices.n));
  j.set("devices", dev);
  return j;
}
ShardedShape ShardedShape::FromJson(const Json& j) {
  ShardedShape s;
  s.dtype = DTypeFromName(j.at("dtype").str);
  for (auto& e : j.at("dims").arr) {
    s.sizes.push_back(e.at("size").as_int());
    std::vector<int> ax;
    for (auto& a : e.at("mesh_axes").arr) ax.push_back(static_cast<int>(a.as_int()));
    s.dim_axes.push_back(ax);
  }
  for (auto& m : j.at("mesh_dims").arr) s.mesh_dims.push_back(static_cast<int>(m.as_int()));
  s.devices.start = static_cast<int>(j.at("devices").at("start").as_int());
  s.devices.n = static_cast<int>(j.at("devices").at("num_devices").as_int());
  return s;
}

bool MeshEquivalent(const ShardedShape& a, const ShardedShape& b) {
  if (a.dtype != b.dtype || a.sizes != b.sizes || a.devices != b.devices) return false;
  for (int i = 0; i < a.devices.n; ++i)
    if (!(a.TileBox(i) == b.TileBox(i))) return false;
  return true;
}

bool NeedsReshard(const ShardedShape& src, const ShardedShape& dst) {
  if (src.IsReplicated() && dst.IsReplicated() && src.devices.Contains(dst.devices)) return false;
  if (src.devices != dst.devices) return true;
  return !MeshEquivalent(src, dst);
}

ShardedShape ResizeSharding(const ShardedShape& s, DeviceRange dst, bool* ok) {
  if (ok) *ok = true;
  if (s.IsReplicated()) return ShardedShape::Replicated(s.dtype, s.sizes, dst);
  // identity permutation: sharded dims use mesh axes in ascending order
  int last = -1;
  bool identity = true;
  for (int d = 0; d < s.rank(); ++d)
    for (int a : s.dim_axes[d]) { if (a < last) identity = false; last = a; }
  ShardedShape out;
  out.dtype = s.dtype;
  out.sizes = s.sizes;
  out.devices = dst;
  if (identity && s.Replication() == 1) {
    int first = -1;
    for (int d = 0; d < s.rank(); ++d) if (s.Shards(d) > 1) { first = d; break; }
    const int src_n = s.devices.n;
    const int64_t scaled = static_cast<int64_t>(s.Shards(first)) * dst.n;
    if (scaled % src_n == 0) {
      const int new_shards = static_cast<int>(scaled / src_n);
      if (new_shards >= 1 && new_shards <= s.sizes[first] && s.sizes[first] % new_shards == 0) {
        // one mesh axis per sharded dim, in order
        out.dim_axes.assign(s.rank(), {});
        for (int d = 0; d < s.rank(); ++d) {
          const int sh = d == first ? new_shards : s.Shards(d);
          if (sh > 1) {
            out.dim_axes[d] = {static_cast<int>(out.mesh_dims.size())};
            out.mesh_dims.push_back(sh);
          }
        }
        if (out.mesh_dims.empty()) out.mesh_dims = {dst.n};
        int mesh = 1;
        for (int m : out.mesh_dims) mesh *= m;
        if (mesh == dst.n) return out;
      }
    }
  }
  if (ok) *ok = false;
  return ShardedShape::Replicated(s.dtype, s.sizes, dst);
}

ShardedShape ReplicateDims(const ShardedShape& s, const std::vector<int>& dims) {
  ShardedShape out = s;
  for (int d : dims) out.dim_axes[d].clear();
  return out;
}

ShardedShape LogicalToPhysical(DType dtype, const std::vector<int64_t>& sizes,
                               const std::vector<std::vector<std::string>>& axes,
                               const std::vector<std::pair<std::string, std::string>>& logical_axes,
                               const std::vector<std::string>& mesh_axis_names,
                               const std::vector<int>& mesh_dims, DeviceRange devices) {
  ShardedShape s;
  s.dtype = dtype;
  s.sizes = sizes;
  s.mesh_dims = mesh_dims;
  s.devices = devices;
  s.dim_axes.assign(sizes.size(), {});
  std::vector<bool> used(mesh_dims.size(), false);
  for (auto& la : logical_axes) {
    int axis = -1;
    for (size_t i = 0; i < mesh_axis_names.size(); ++i) if (mesh_axis_names[i] == la.second) axis = static_cast<int>(i);
    // an axis with a single device shards nothing: listing it would only make equal layouts
    // look different
    if (axis < 0 || used[axis] || mesh_dims[axis] == 1) continue;
    for (size_t d = 0; d < sizes.size() && d < axes.size(); ++d) {
      if (std::find(axes[d].begin(), axes[d].end(), la.first) == axes[d].end()) continue;
      const int64_t shards = static_cast<int64_t>(s.Shards(static_cast<int>(d))) * mesh_dims[axis];
      if (shards <= sizes[d] && sizes[d] % shards == 0) {
        s.dim_axes[d].push_back(axis);
        used[axis] = true;
        break;
      }
    }
  }
  for (auto& ax : s.dim_axes) std::sort(ax.begin(), ax.end());
  return s;
}

int64_t ReshardPlan::BytesOverLinks() const {
  int64_t b = 0;
  for (auto& c : chunks) if (c.src_device != c.dst_device) b += c.box.Volume();
  return b * static_cast<int64_t>(DTypeSize(src.dtype));
}
int64_t ReshardPlan::BytesTotal() const {
  int64_t b = 0;
  for (auto& c : chunks) b += c.box.Volume();
  return b * static_cast<int64_t>(DTypeSize(src.dtype));
}

ReshardPlan PlanReshard(const ShardedShape& src, const ShardedShape& dst) {
  if (src.sizes != dst.sizes || src.dtype != dst.dtype)
    throw std::runtime_error("reshard: source and destination describe different arrays");
  ReshardPlan plan;
  plan.src = src;
  plan.dst = dst;
  // unique source tiles -> the replicas (device ordinals) holding them
  std::vector<Box> tiles;
  std::vector<std::vector<int>> holders;
  for (int i = 0; i < src.devices.n; ++i) {
    Box b = src.TileBox(i);
    size_t t = 0;
    for (; t < tiles.size(); ++t) if (tiles[t] == b) break;
    if (t == tiles.size()) { tiles.push_back(b); holders.emplace_back(); }
    holders[t].push_back(i);
  }
  for (int j = 0; j < dst.devices.n; ++j) {
    const int dst_dev = dst.devices[j];
    const Box want = dst.TileBox(j);
    for (size_t t = 0; t < tiles.size(); ++t) {
      Box inter = Box::Intersect(want, tiles[t]);
      if (inter.Empty()) continue;
      // choose the replica: the destination itself if it holds the tile, else round-robin
      int chosen = -1;
      for (int h : holders[t]) if (src.devices[h] == dst_dev) chosen = h;
      if (chosen < 0) chosen = holders[t][j % holders[t].size()];
      ReshardChunk c;
      c.src_device = src.devices[chosen];
      c.dst_device = dst_dev;
      c.box = inter;
      c.src_offset.resize(inter.lo.size());
      c.dst_offset.resize(inter.lo.size());
      for (size_t d = 0; d < inter.lo.size(); ++d) {
        c.src_offset[d] = inter.lo[d] - tiles[t].lo[d];
        c.dst_offset[d] = inter.lo[d] - want.lo[d];
      }
      plan.chunks.push_back(std::move(c));
    }
  }
  return plan;
}

}  // namespace mmg
