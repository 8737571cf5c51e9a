// Native parquet reader on the Arrow C++ / parquet-cpp libraries that ship inside the pyarrow wheel.
//
// Exposes, as plain C entry points: file metadata (rows, row groups, flat column names and physical types),
// one BYTE_ARRAY column of one row group as a packed byte buffer + offsets (the document stream of the
// pre-training loader), and a row group or a whole file rendered as JSON lines (flat schemas: booleans,
// integers, floats, strings; nulls become `null`).  Every entry point catches C++ exceptions and returns a
// negative status with the message copied into the caller's buffer.
//
// The reference's counterpart links the same libraries (cc/src/tyr_parquet.cpp:88-557: list files, metadata,
// row-group text column, whole file / row group to JSON lines).
#include <parquet/api/reader.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#define TYR_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct Handle {
  std::unique_ptr<parquet::ParquetFileReader> reader;
  std::shared_ptr<parquet::FileMetaData> meta;
};

void set_err(char* err, int errlen, const std::string& msg) {
  if (err && errlen > 0) {
    std::snprintf(err, static_cast<size_t>(errlen), "%s", msg.c_str());
  }
}

int find_column(const Handle& h, const char* name) {
  const auto* schema = h.meta->schema();
  for (int i = 0; i < schema->num_columns(); ++i)
    if (schema->Column(i)->path()->ToDotString() == name) return i;
  return -1;
}

void json_escape(std::string& out, const uint8_t* p, uint32_t n) {
  out.push_back('"');
  for (uint32_t i = 0; i < n; ++i) {
    const uint8_t c = p[i];
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      case '\b': out += "\\b"; break;
      case '\f': out += "\\f"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          std::snprintf(buf, sizeof(buf), "\\u%04x", c);
          out += buf;
        } else {
          out.push_back(static_cast<char>(c));
        }
    }
  }
  out.push_back('"');
}

// One column of one row group rendered to JSON scalars, one string per row.
template <typename ReaderT, typename ValueT, typename Fmt>
void read_cells(parquet::ColumnReader* col, int16_t max_def, int64_t rows, std::vector<std::string>& cells, Fmt fmt) {
  auto* r = static_cast<ReaderT*>(col);
  constexpr int64_t kBatch = 4096;
  std::vector<int16_t> def(kBatch);
  std::unique_ptr<ValueT[]> vals(new ValueT[kBatch]);
  cells.clear();
  cells.reserve(static_cast<size_t>(rows));
  while (r->HasNext()) {
    int64_t got = 0;
    const int64_t levels = r->ReadBatch(kBatch, max_def > 0 ? def.data() : nullptr, nullptr, vals.get(), &got);
    if (levels == 0 && got == 0) break;
    const int64_t n = max_def > 0 ? levels : got;
    int64_t vi = 0;
    for (int64_t i = 0; i < n; ++i) {
      if (max_def > 0 && def[static_cast<size_t>(i)] < max_def) {
        cells.emplace_back("null");
      } else {
        std::string s;
        fmt(s, vals[static_cast<size_t>(vi++)]);
        cells.push_back(std::move(s));
      }
    }
  }
}

void fmt_double(std::string& s, double v) {
  if (!std::isfinite(v)) { s = "null"; return; }
  char buf[40];
  std::snprintf(buf, sizeof(buf), "%.17g", v);
  s = buf;
}

int row_group_to_json(Handle& h, int g, std::string& out, std::string& why) {
  const auto* schema = h.meta->schema();
  const int ncol = schema->num_columns();
  auto rg = h.reader->RowGroup(g);
  const int64_t rows = rg->metadata()->num_rows();
  std::vector<std::vector<std::string>> cols(static_cast<size_t>(ncol));
  std::vector<std::string> names(static_cast<size_t>(ncol));
  for (int c = 0; c < ncol; ++c) {
    const auto* d = schema->Column(c);
    if (d->max_repetition_level() > 0) {
      why = "nested / repeated column '" + d->path()->ToDotString() + "' is not supported by the native JSON path";
      return -3;
    }
    std::string nm;
    const std::string dotted = d->path()->ToDotString();
    json_escape(nm, reinterpret_cast<const uint8_t*>(dotted.data()), static_cast<uint32_t>(dotted.size()));
    names[static_cast<size_t>(c)] = nm;
    auto col = rg->Column(c);
    const int16_t md = d->max_definition_level();
    auto& cells = cols[static_cast<size_t>(c)];
    switch (d->physical_type()) {
      case parquet::Type::BOOLEAN:
        read_cells<parquet::BoolReader, bool>(col.get(), md, rows, cells, [](std::string& s, bool v) { s = v ? "true" : "false"; });
        break;
      case parquet::Type::INT32:
        read_cells<parquet::Int32Reader, int32_t>(col.get(), md, rows, cells, [](std::string& s, int32_t v) { s = std::to_string(v); });
        break;
      case parquet::Type::INT64:
        read_cells<parquet::Int64Reader, int64_t>(col.get(), md, rows, cells, [](std::string& s, int64_t v) { s = std::to_string(v); });
        break;
      case parquet::Type::FLOAT:
        read_cells<parquet::FloatReader, float>(col.get(), md, rows, cells, [](std::string& s, float v) { fmt_double(s, v); });
        break;
      case parquet::Type::DOUBLE:
        read_cells<parquet::DoubleReader, double>(col.get(), md, rows, cells, [](std::string& s, double v) { fmt_double(s, v); });
        break;
      case parquet::Type::BYTE_ARRAY:
        read_cells<parquet::ByteArrayReader, parquet::ByteArray>(col.get(), md, rows, cells,
                                                                [](std::string& s, const parquet::ByteArray& v) { json_escape(s, v.ptr, v.len); });
        break;
      default:
        why = "column '" + dotted + "' has a physical type the native JSON path does not render";
        return -3;
    }
    if (static_cast<int64_t>(cells.size()) != rows) {
      why = "column '" + dotted + "' produced " + std::to_string(cells.size()) + " cells for " + std::to_string(rows) + " rows";
      return -4;
    }
  }
  for (int64_t r = 0; r < rows; ++r) {
    out.push_back('{');
    for (int c = 0; c < ncol; ++c) {
      if (c) out.push_back(',');
      out += names[static_cast<size_t>(c)];
      out.push_back(':');
      out += cols[static_cast<size_t>(c)][static_cast<size_t>(r)];
    }
    out += "}\n";
  }
  return 0;
}

char* dup_buffer(const std::string& s) {
  char* p = static_cast<char*>(std::malloc(s.size() + 1));
  if (p) {
    std::memcpy(p, s.data(), s.size());
    p[s.size()] = 0;
  }
  return p;
}

}  // namespace

#define TYR_GUARD(...)                                     \
  try {                                                    \
    __VA_ARGS__                                            \
  } catch (const std::exception& e) {                      \
    set_err(err, errlen, e.what());                        \
    return -1;                                             \
  } catch (...) {                                          \
    set_err(err, errlen, "unknown C++ exception");         \
    return -1;                                             \
  }

TYR_EXPORT int tyr_parquet_open(const char* path, void** out, char* err, int errlen) {
  TYR_GUARD({
    auto h = std::make_unique<Handle>();
    h->reader = parquet::ParquetFileReader::OpenFile(path, /*memory_map=*/true);
    h->meta = h->reader->metadata();
    *out = h.release();
    return 0;
  })
}

TYR_EXPORT void tyr_parquet_close(void* handle) { delete static_cast<Handle*>(handle); }

// info: {rows, row groups, leaf columns}
TYR_EXPORT int tyr_parquet_info(void* handle, long long* info) {
  auto* h = static_cast<Handle*>(handle);
  info[0] = h->meta->num_rows();
  info[1] = h->meta->num_row_groups();
  info[2] = h->meta->schema()->num_columns();
  return 0;
}

TYR_EXPORT long long tyr_parquet_row_group_rows(void* handle, int g) {
  auto* h = static_cast<Handle*>(handle);
  if (g < 0 || g >= h->meta->num_row_groups()) return -1;
  return h->meta->RowGroup(g)->num_rows();
}

// Dotted path of leaf column `i` copied into `buf`; returns the physical type tag (parquet::Type) or -1.
TYR_EXPORT int tyr_parquet_column(void* handle, int i, char* buf, int buflen) {
  auto* h = static_cast<Handle*>(handle);
  const auto* schema = h->meta->schema();
  if (i < 0 || i >= schema->num_columns()) return -1;
  std::snprintf(buf, static_cast<size_t>(buflen), "%s", schema->Column(i)->path()->ToDotString().c_str());
  return static_cast<int>(schema->Column(i)->physical_type());
}

// One BYTE_ARRAY column of one row group: *data (malloc'd, all values back to back), *offsets (malloc'd, n + 1
// entries; a null row has equal neighbours and valid[i] == 0), *valid (malloc'd, n bytes).  Free with tyr_parquet_free.
TYR_EXPORT int tyr_parquet_read_text(void* handle, int g, const char* column, char** data, long long** offsets,
                                     unsigned char** valid, long long* n_rows, char* err, int errlen) {
  TYR_GUARD({
    auto* h = static_cast<Handle*>(handle);
    if (g < 0 || g >= h->meta->num_row_groups()) {
      set_err(err, errlen, "row group out of range");
      return -2;
    }
    const int c = find_column(*h, column);
    if (c < 0) {
      set_err(err, errlen, std::string("no column named '") + column + "'");
      return -2;
    }
    const auto* d = h->meta->schema()->Column(c);
    if (d->physical_type() != parquet::Type::BYTE_ARRAY || d->max_repetition_level() > 0) {
      set_err(err, errlen, std::string("column '") + column + "' is not a flat string / binary column");
      return -3;
    }
    auto rg = h->reader->RowGroup(g);
    auto col = rg->Column(c);
    auto* r = static_cast<parquet::ByteArrayReader*>(col.get());
    const int16_t md = d->max_definition_level();
    constexpr int64_t kBatch = 1024;
    std::vector<int16_t> def(kBatch);
    std::vector<parquet::ByteArray> vals(kBatch);
    std::string bytes;
    std::vector<long long> off{0};
    std::vector<unsigned char> ok;
    while (r->HasNext()) {
      int64_t got = 0;
      const int64_t levels = r->ReadBatch(kBatch, md > 0 ? def.data() : nullptr, nullptr, vals.data(), &got);
      if (levels == 0 && got == 0) break;
      const int64_t n = md > 0 ? levels : got;
      int64_t vi = 0;
      for (int64_t i = 0; i < n; ++i) {
        const bool present = !(md > 0 && def[static_cast<size_t>(i)] < md);
        if (present) {
          const auto& v = vals[static_cast<size_t>(vi++)];
          bytes.append(reinterpret_cast<const char*>(v.ptr), v.len);
        }
        ok.push_back(present ? 1 : 0);
        off.push_back(static_cast<long long>(bytes.size()));
      }
    }
    const size_t n = ok.size();
    *data = dup_buffer(bytes);
    *offsets = static_cast<long long*>(std::malloc((n + 1) * sizeof(long long)));
    *valid = static_cast<unsigned char*>(std::malloc(std::max<size_t>(n, 1)));
    if (!*data || !*offsets || !*valid) {
      set_err(err, errlen, "out of memory");
      return -5;
    }
    std::memcpy(*offsets, off.data(), (n + 1) * sizeof(long long));
    if (n) std::memcpy(*valid, ok.data(), n);
    *n_rows = static_cast<long long>(n);
    return 0;
  })
}

// JSON lines of one row group (g >= 0) or of the whole file (g < 0) in a malloc'd, NUL-terminated buffer.
TYR_EXPORT int tyr_parquet_to_json_lines(void* handle, int g, char** out, long long* out_len, char* err, int errlen) {
  TYR_GUARD({
    auto* h = static_cast<Handle*>(handle);
    const int ng = h->meta->num_row_groups();
    if (g >= ng) {
      set_err(err, errlen, "row group out of range");
      return -2;
    }
    std::string text, why;
    for (int i = (g < 0 ? 0 : g); i < (g < 0 ? ng : g + 1); ++i) {
      const int rc = row_group_to_json(*h, i, text, why);
      if (rc != 0) {
        set_err(err, errlen, why);
        return rc;
      }
    }
    *out = dup_buffer(text);
    if (!*out) {
      set_err(err, errlen, "out of memory");
      return -5;
    }
    *out_len = static_cast<long long>(text.size());
    return 0;
  })
}

TYR_EXPORT void tyr_parquet_free(void* p) { std::free(p); }
