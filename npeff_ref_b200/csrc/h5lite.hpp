// A small, self-contained HDF5 codec for exactly what the D-NPEFF path reads and
// writes (no libhdf5 exists where this is built).  Written from the public "HDF5
// File Format Specification".
//
// Writer: the layout H5Fcreate(H5P_DEFAULT) produces -- superblock version 0,
//   old-style groups (symbol-table message -> v1 B-tree "TREE" -> symbol node
//   "SNOD", names in a local heap "HEAP"), version-1 object headers, contiguous
//   little-endian datasets, version-1 attribute messages.  This is what the
//   reference writes (src/io/nmf_decomp_h5.h:38-89) and what
//   npeff/decomp/decomps.py:55-71 reads back through h5py.
// Reader: that same layout (what h5py's default File(..., "w") produces for
//   npeff/fishers/d_pefs_computer.py:235-251), plus superblock 2/3 with
//   version-2 object headers and compact link messages (libver="latest").
//   Datasets must be contiguous or compact; chunked or filtered datasets, dense
//   (fractal-heap) groups and external links are rejected with a message.
#pragma once
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace h5lite {

struct Error : std::runtime_error {
    explicit Error(const std::string& m) : std::runtime_error(m) {}
};

enum class TypeClass { Int = 0, Float = 1, Other = 2 };

struct DType {
    TypeClass cls = TypeClass::Int;
    int size = 4;          // bytes
    bool is_signed = true;
    bool big_endian = false;
    static DType f32() { return {TypeClass::Float, 4, true, false}; }
    static DType i32() { return {TypeClass::Int, 4, true, false}; }
    static DType i64() { return {TypeClass::Int, 8, true, false}; }
};

constexpr uint64_t kUndef = 0xFFFFFFFFFFFFFFFFull;

// ============================================================================
// Writer
// ============================================================================
class Writer {
  public:
    struct Attr {
        std::string name;
        DType type;
        std::vector<uint64_t> dims;  // empty = scalar
        std::vector<uint8_t> data;
    };

    explicit Writer(const std::string& path) : path_(path) {
        root_.reset(new Node());
        root_->is_group = true;
    }

    void add_group(const std::string& path) { lookup(path, true); }

    // `data` must stay valid until finish().
    void add_dataset(const std::string& path, DType type, const std::vector<uint64_t>& dims,
                     const void* data) {
        Node* n = lookup(path, true);
        if (!n->children.empty()) throw Error("h5lite: " + path + " is a group");
        n->is_group = false;
        n->type = type;
        n->dims = dims;
        n->data = data;
    }

    void add_attr(const std::string& object_path, const std::string& name, DType type,
                  const std::vector<uint64_t>& dims, const void* data) {
        Node* n = lookup(object_path, false);
        Attr a;
        a.name = name;
        a.type = type;
        a.dims = dims;
        uint64_t count = 1;
        for (uint64_t d : dims) count *= d;
        a.data.assign((const uint8_t*)data, (const uint8_t*)data + count * type.size);
        n->attrs.push_back(a);
    }

    void finish() {
        // 1. lay the file out
        uint64_t pos = 96;  // superblock
        assign(root_.get(), pos);
        uint64_t eof = pos;
        // 2. write it
        FILE* f = fopen(path_.c_str(), "wb");
        if (!f) throw Error("h5lite: cannot create " + path_);
        try {
            std::vector<uint8_t> sb = superblock(eof);
            put(f, 0, sb.data(), sb.size());
            emit(f, root_.get());
            // make the file exactly `eof` bytes long
            if (fseeko(f, 0, SEEK_END) != 0) throw Error("h5lite: seek failed");
            uint64_t len = (uint64_t)ftello(f);
            if (len < eof) {
                std::vector<uint8_t> z((size_t)(eof - len), 0);
                put(f, len, z.data(), z.size());
            }
        } catch (...) {
            fclose(f);
            throw;
        }
        if (fclose(f) != 0) throw Error("h5lite: write to " + path_ + " failed");
    }

  private:
    struct Node {
        bool is_group = true;
        std::map<std::string, std::unique_ptr<Node>> children;  // std::map: strcmp order
        std::vector<Attr> attrs;
        DType type;
        std::vector<uint64_t> dims;
        const void* data = nullptr;
        // layout
        uint64_t header_addr = 0, btree_addr = 0, heap_addr = 0, heap_data_addr = 0, snod_addr = 0,
                 data_addr = 0, data_bytes = 0, heap_data_size = 0;
        std::vector<uint8_t> header;  // encoded object header
        std::map<std::string, uint64_t> name_off;
    };

    static constexpr int kLeafK = 4, kInternalK = 16;
    static constexpr uint64_t kBtreeNodeSize = 24 + (2 * kInternalK + 1) * 8 + 2 * kInternalK * 8;  // 544
    static constexpr uint64_t kSnodSize = 8 + 2 * kLeafK * 40;                                       // 328

    std::string path_;
    std::unique_ptr<Node> root_;

    static uint64_t align8(uint64_t x) { return (x + 7) & ~7ull; }

    Node* lookup(const std::string& path, bool create) {
        Node* cur = root_.get();
        size_t i = 0;
        while (i < path.size()) {
            while (i < path.size() && path[i] == '/') i++;
            size_t j = i;
            while (j < path.size() && path[j] != '/') j++;
            if (j == i) break;
            std::string part = path.substr(i, j - i);
            auto it = cur->children.find(part);
            if (it == cur->children.end()) {
                if (!create) throw Error("h5lite: no object " + path);
                if (!cur->is_group) throw Error("h5lite: " + part + " is under a dataset");
                if (cur->children.size() >= (size_t)(2 * kLeafK))
                    throw Error("h5lite: more than 8 links in one group is not supported");
                it = cur->children.emplace(part, std::unique_ptr<Node>(new Node())).first;
            }
            cur = it->second.get();
            i = j;
        }
        return cur;
    }

    // ---- little-endian byte buffer helpers ------------------------------------
    static void u8(std::vector<uint8_t>& b, uint64_t v) { b.push_back((uint8_t)v); }
    static void u16(std::vector<uint8_t>& b, uint64_t v) { for (int i = 0; i < 2; i++) b.push_back((uint8_t)(v >> (8 * i))); }
    static void u32(std::vector<uint8_t>& b, uint64_t v) { for (int i = 0; i < 4; i++) b.push_back((uint8_t)(v >> (8 * i))); }
    static void u64(std::vector<uint8_t>& b, uint64_t v) { for (int i = 0; i < 8; i++) b.push_back((uint8_t)(v >> (8 * i))); }
    static void pad8(std::vector<uint8_t>& b) { while (b.size() % 8) b.push_back(0); }

    static std::vector<uint8_t> enc_dtype(const DType& t) {
        std::vector<uint8_t> b;
        if (t.cls == TypeClass::Int) {
            u8(b, 0x10 | 0);                        // version 1, class 0 (fixed point)
            u8(b, (t.is_signed ? 0x08 : 0) | 0);    // little-endian, pad 0, signed
            u8(b, 0); u8(b, 0);
            u32(b, t.size);
            u16(b, 0);                              // bit offset
            u16(b, t.size * 8);                     // precision
        } else {
            u8(b, 0x10 | 1);                        // version 1, class 1 (floating point)
            u8(b, 0x20);                            // little-endian, mantissa normalisation 2 (implied msb)
            u8(b, t.size == 4 ? 31 : 63);           // sign bit position
            u8(b, 0);
            u32(b, t.size);
            u16(b, 0);                              // bit offset
            u16(b, t.size * 8);                     // precision
            if (t.size == 4) { u8(b, 23); u8(b, 8); u8(b, 0); u8(b, 23); u32(b, 127); }
            else { u8(b, 52); u8(b, 11); u8(b, 0); u8(b, 52); u32(b, 1023); }
        }
        return b;
    }

    static std::vector<uint8_t> enc_dspace(const std::vector<uint64_t>& dims) {
        std::vector<uint8_t> b;
        u8(b, 1);                 // version 1
        u8(b, dims.size());       // rank
        u8(b, 0);                 // flags: no max dims
        u8(b, 0); u32(b, 0);      // reserved
        for (uint64_t d : dims) u64(b, d);
        return b;
    }

    static void msg(std::vector<uint8_t>& h, int type, const std::vector<uint8_t>& body, int& count) {
        std::vector<uint8_t> d = body;
        pad8(d);
        u16(h, type);
        u16(h, d.size());
        u8(h, 0);                 // flags
        u8(h, 0); u8(h, 0); u8(h, 0);
        h.insert(h.end(), d.begin(), d.end());
        count++;
    }

    static void attr_msgs(std::vector<uint8_t>& h, const std::vector<Attr>& attrs, int& count) {
        for (const Attr& a : attrs) {
            std::vector<uint8_t> dt = enc_dtype(a.type), ds = enc_dspace(a.dims), b;
            u8(b, 1); u8(b, 0);                       // version 1
            u16(b, a.name.size() + 1);
            u16(b, dt.size());
            u16(b, ds.size());
            b.insert(b.end(), a.name.begin(), a.name.end());
            b.push_back(0);
            pad8(b);
            b.insert(b.end(), dt.begin(), dt.end());
            pad8(b);
            b.insert(b.end(), ds.begin(), ds.end());
            pad8(b);
            b.insert(b.end(), a.data.begin(), a.data.end());
            msg(h, 0x000C, b, count);
        }
    }

    static std::vector<uint8_t> finish_header(const std::vector<uint8_t>& msgs, int count) {
        std::vector<uint8_t> h;
        u8(h, 1); u8(h, 0);       // version 1
        u16(h, count);
        u32(h, 1);                // object reference count
        u32(h, msgs.size());      // size of the message block
        u32(h, 0);                // pad the prefix to 16 bytes
        h.insert(h.end(), msgs.begin(), msgs.end());
        return h;
    }

    // Assigns addresses depth first; `pos` is the next free (8-aligned) offset.
    void assign(Node* n, uint64_t& pos) {
        if (n->is_group) {
            // heap contents: "" at 0, then the link names
            uint64_t off = 8;
            for (auto& kv : n->children) {
                n->name_off[kv.first] = off;
                off += align8(kv.first.size() + 1);
            }
            n->heap_data_size = off + 16;  // names + one free block closing the segment
            n->header_addr = pos;
            // header: one symbol-table message (16 bytes) + attributes; sized after
            // the children only in its contents, not in its length
            std::vector<uint8_t> m;
            int count = 0;
            msg(m, 0x0011, std::vector<uint8_t>(16, 0), count);
            attr_msgs(m, n->attrs, count);
            uint64_t hsize = 16 + m.size();
            pos = align8(pos + hsize);
            n->btree_addr = pos; pos += kBtreeNodeSize;
            n->heap_addr = pos; pos += 32;
            n->heap_data_addr = pos; pos = align8(pos + n->heap_data_size);
            n->snod_addr = pos; pos += kSnodSize;
            for (auto& kv : n->children) assign(kv.second.get(), pos);
            // now the real header
            std::vector<uint8_t> st;
            u64(st, n->btree_addr);
            u64(st, n->heap_addr);
            std::vector<uint8_t> mm;
            count = 0;
            msg(mm, 0x0011, st, count);
            attr_msgs(mm, n->attrs, count);
            n->header = finish_header(mm, count);
        } else {
            uint64_t count_el = 1;
            for (uint64_t d : n->dims) count_el *= d;
            n->data_bytes = count_el * n->type.size;
            n->header_addr = pos;
            auto build = [&](uint64_t data_addr) {
                std::vector<uint8_t> m;
                int count = 0;
                msg(m, 0x0001, enc_dspace(n->dims), count);
                msg(m, 0x0003, enc_dtype(n->type), count);
                std::vector<uint8_t> fill;
                u8(fill, 2);   // version 2
                u8(fill, 1);   // space allocation time: early
                u8(fill, 0);   // fill value write time: on allocation
                u8(fill, 1);   // fill value defined ...
                u32(fill, 0);  // ... with size 0: the default (zero) fill value
                msg(m, 0x0005, fill, count);
                std::vector<uint8_t> lay;
                u8(lay, 3);    // version 3
                u8(lay, 1);    // contiguous
                u64(lay, n->data_bytes ? data_addr : kUndef);
                u64(lay, n->data_bytes);
                msg(m, 0x0008, lay, count);
                attr_msgs(m, n->attrs, count);
                return finish_header(m, count);
            };
            uint64_t hsize = build(0).size();
            pos = align8(pos + hsize);
            n->data_addr = pos;
            pos = align8(pos + n->data_bytes);
            n->header = build(n->data_addr);
        }
    }

    std::vector<uint8_t> superblock(uint64_t eof) {
        std::vector<uint8_t> b;
        const uint8_t sig[8] = {0x89, 'H', 'D', 'F', '\r', '\n', 0x1a, '\n'};
        b.insert(b.end(), sig, sig + 8);
        u8(b, 0);  // superblock version
        u8(b, 0);  // free-space storage version
        u8(b, 0);  // root group symbol table entry version
        u8(b, 0);
        u8(b, 0);  // shared header message format version
        u8(b, 8);  // size of offsets
        u8(b, 8);  // size of lengths
        u8(b, 0);
        u16(b, kLeafK);
        u16(b, kInternalK);
        u32(b, 0);       // file consistency flags
        u64(b, 0);       // base address
        u64(b, kUndef);  // free-space info
        u64(b, eof);     // end of file address
        u64(b, kUndef);  // driver information block
        // root group symbol table entry
        u64(b, 0);                    // link name offset
        u64(b, root_->header_addr);
        u32(b, 1);                    // cache type 1: group, scratch holds B-tree and heap
        u32(b, 0);
        u64(b, root_->btree_addr);
        u64(b, root_->heap_addr);
        return b;
    }

    static void put(FILE* f, uint64_t at, const void* p, size_t n) {
        if (n == 0) return;
        if (fseeko(f, (off_t)at, SEEK_SET) != 0 || fwrite(p, 1, n, f) != n)
            throw Error("h5lite: write failed");
    }

    void emit(FILE* f, Node* n) {
        put(f, n->header_addr, n->header.data(), n->header.size());
        if (!n->is_group) {
            put(f, n->data_addr, n->data, (size_t)n->data_bytes);
            return;
        }
        // B-tree node: one leaf-level entry pointing at the symbol node
        std::vector<uint8_t> b;
        b.insert(b.end(), {'T', 'R', 'E', 'E'});
        u8(b, 0);                 // node type 0: group
        u8(b, 0);                 // level 0
        u16(b, 1);                // entries used
        u64(b, kUndef);           // left sibling
        u64(b, kUndef);           // right sibling
        u64(b, 0);                // key 0: heap offset of ""
        u64(b, n->snod_addr);     // child 0
        uint64_t last = 0;
        if (!n->children.empty()) last = n->name_off[n->children.rbegin()->first];
        u64(b, last);             // key 1: heap offset of the largest name in child 0
        b.resize((size_t)kBtreeNodeSize, 0);
        put(f, n->btree_addr, b.data(), b.size());
        // local heap
        std::vector<uint8_t> h;
        h.insert(h.end(), {'H', 'E', 'A', 'P'});
        u8(h, 0); u8(h, 0); u8(h, 0); u8(h, 0);
        u64(h, n->heap_data_size);
        u64(h, n->heap_data_size - 16);  // head of the free list
        u64(h, n->heap_data_addr);
        put(f, n->heap_addr, h.data(), h.size());
        std::vector<uint8_t> d((size_t)n->heap_data_size, 0);
        for (auto& kv : n->children) memcpy(d.data() + n->name_off[kv.first], kv.first.data(), kv.first.size());
        {
            std::vector<uint8_t> fb;
            u64(fb, 1);           // no next free block
            u64(fb, 16);          // size of this free block
            memcpy(d.data() + n->heap_data_size - 16, fb.data(), 16);
        }
        put(f, n->heap_data_addr, d.data(), d.size());
        // symbol node
        std::vector<uint8_t> s;
        s.insert(s.end(), {'S', 'N', 'O', 'D'});
        u8(s, 1); u8(s, 0);
        u16(s, n->children.size());
        for (auto& kv : n->children) {
            Node* c = kv.second.get();
            u64(s, n->name_off[kv.first]);
            u64(s, c->header_addr);
            if (c->is_group) {
                u32(s, 1); u32(s, 0);
                u64(s, c->btree_addr);
                u64(s, c->heap_addr);
            } else {
                u32(s, 0); u32(s, 0);
                u64(s, 0); u64(s, 0);
            }
        }
        s.resize((size_t)kSnodSize, 0);
        put(f, n->snod_addr, s.data(), s.size());
        for (auto& kv : n->children) emit(f, kv.second.get());
    }
};

// ============================================================================
// Reader
// ============================================================================
struct Dataspace {
    std::vector<uint64_t> dims;  // empty = scalar
    uint64_t count() const {
        uint64_t c = 1;
        for (uint64_t d : dims) c *= d;
        return c;
    }
};

struct AttrInfo {
    DType type;
    Dataspace space;
    std::vector<uint8_t> data;
};

struct ObjectInfo {
    bool is_group = false;
    // group
    uint64_t btree_addr = kUndef, heap_addr = kUndef;
    std::map<std::string, uint64_t> links;  // from link messages (new-style compact groups)
    bool has_link_info_dense = false;
    // dataset
    bool has_type = false, has_space = false, has_layout = false;
    DType type;
    Dataspace space;
    int layout_class = -1;  // 0 compact, 1 contiguous, 2 chunked
    uint64_t data_addr = kUndef, data_size = 0;
    std::vector<uint8_t> compact;
    bool filtered = false;
    std::map<std::string, AttrInfo> attrs;
};

class Reader {
  public:
    explicit Reader(const std::string& path) : path_(path) {
        f_ = fopen(path.c_str(), "rb");
        if (!f_) throw Error("h5lite: cannot open " + path);
        try {
            fseeko(f_, 0, SEEK_END);
            file_size_ = (uint64_t)ftello(f_);
            read_superblock();
        } catch (...) {
            fclose(f_);
            f_ = nullptr;
            throw;
        }
    }
    ~Reader() {
        if (f_) fclose(f_);
    }
    Reader(const Reader&) = delete;
    Reader& operator=(const Reader&) = delete;

    // Object header address of `path` ("data/fisher/values").
    uint64_t find(const std::string& path) {
        uint64_t cur = root_addr_;
        size_t i = 0;
        while (i < path.size()) {
            while (i < path.size() && path[i] == '/') i++;
            size_t j = i;
            while (j < path.size() && path[j] != '/') j++;
            if (j == i) break;
            std::string part = path.substr(i, j - i);
            ObjectInfo o = object(cur);
            if (!o.is_group) throw Error("h5lite: " + path + ": '" + part + "' is looked up in a non-group");
            cur = lookup_link(o, part, path);
            i = j;
        }
        return cur;
    }

    ObjectInfo object(uint64_t addr) {
        ObjectInfo o;
        uint8_t sig[4];
        rd(addr, sig, 4);
        if (memcmp(sig, "OHDR", 4) == 0) parse_v2_header(addr, o);
        else parse_v1_header(addr, o);
        if (o.btree_addr != kUndef || !o.links.empty() || o.has_link_info_dense) o.is_group = true;
        if (!o.has_layout && !o.has_type) o.is_group = true;  // an empty new-style group
        return o;
    }

    ObjectInfo dataset(const std::string& path) {
        ObjectInfo o = object(find(path));
        if (!(o.has_type && o.has_space && o.has_layout)) throw Error("h5lite: " + path + " is not a dataset");
        if (o.type.cls == TypeClass::Other)
            throw Error("h5lite: " + path + ": only integer and floating-point datasets are supported");
        if (o.filtered) throw Error("h5lite: " + path + ": filtered (compressed) datasets are not supported");
        if (o.layout_class == 2) throw Error("h5lite: " + path + ": chunked datasets are not supported");
        return o;
    }

    // Reads the leading [rows x cols] block of a rank-2 dataset (or the leading
    // `rows` of a rank-1 one, cols = 1) into `out`, converting to `want`.
    void read_leading(const ObjectInfo& o, uint64_t rows, uint64_t cols, DType want, void* out) {
        read_block(o, 0, rows, cols, want, out);
    }

    // Rows [row0, row0 + rows) and the leading `cols` columns of a rank-2 dataset (a
    // rank-1 one: cols = 1) into `out`, converting to `want`.  When the stored type is
    // the wanted one the bytes go straight from the file into `out`.
    void read_block(const ObjectInfo& o, uint64_t row0, uint64_t rows, uint64_t cols, DType want, void* out) {
        uint64_t full_rows = 1, full_cols = 1;
        if (o.space.dims.size() == 1) { full_rows = o.space.dims[0]; full_cols = 1; }
        else if (o.space.dims.size() == 2) { full_rows = o.space.dims[0]; full_cols = o.space.dims[1]; }
        else if (!o.space.dims.empty()) throw Error("h5lite: rank > 2 datasets are not supported");
        if (row0 + rows > full_rows || cols > full_cols) throw Error("h5lite: requested block exceeds the dataset");
        if (rows == 0 || cols == 0) return;
        const size_t es = (size_t)o.type.size;
        uint8_t* dst = (uint8_t*)out;
        const bool same = !o.type.big_endian && o.type.cls == want.cls && o.type.size == want.size;
        if (same) {
            if (cols == full_cols) {
                raw(o, (row0 * full_cols) * es, dst, (size_t)(rows * cols * es));
            } else {
                for (uint64_t r = 0; r < rows; r++)
                    raw(o, ((row0 + r) * full_cols) * es, dst + (size_t)(r * cols * es), (size_t)(cols * es));
            }
            return;
        }
        const uint64_t chunk_rows = std::max<uint64_t>(1, (64ull << 20) / std::max<uint64_t>(1, cols * es));
        std::vector<uint8_t> buf;
        for (uint64_t r0 = 0; r0 < rows; r0 += chunk_rows) {
            uint64_t nr = std::min(chunk_rows, rows - r0);
            buf.resize((size_t)(nr * cols * es));
            if (cols == full_cols) {
                raw(o, ((row0 + r0) * full_cols) * es, buf.data(), buf.size());
            } else {
                for (uint64_t r = 0; r < nr; r++)
                    raw(o, ((row0 + r0 + r) * full_cols) * es, buf.data() + (size_t)(r * cols * es), (size_t)(cols * es));
            }
            convert(buf.data(), o.type, dst + (size_t)(r0 * cols * want.size), want, nr * cols);
        }
    }

    static void convert(const uint8_t* src, const DType& st, uint8_t* dst, const DType& dt, uint64_t count) {
        if (st.big_endian) throw Error("h5lite: big-endian data is not supported");
        if (st.cls == TypeClass::Other) throw Error("h5lite: cannot convert a non-numeric datatype");
        if (st.cls == dt.cls && st.size == dt.size) {
            memcpy(dst, src, (size_t)(count * st.size));
            return;
        }
        for (uint64_t i = 0; i < count; i++) {
            double fv = 0;
            int64_t iv = 0;
            const uint8_t* s = src + i * st.size;
            if (st.cls == TypeClass::Float) {
                if (st.size == 4) { float x; memcpy(&x, s, 4); fv = x; }
                else if (st.size == 8) { memcpy(&fv, s, 8); }
                else throw Error("h5lite: unsupported float size");
                iv = (int64_t)fv;
            } else {
                if (st.size == 1) iv = st.is_signed ? (int64_t)(int8_t)s[0] : (int64_t)s[0];
                else if (st.size == 2) { uint16_t x; memcpy(&x, s, 2); iv = st.is_signed ? (int64_t)(int16_t)x : (int64_t)x; }
                else if (st.size == 4) { uint32_t x; memcpy(&x, s, 4); iv = st.is_signed ? (int64_t)(int32_t)x : (int64_t)x; }
                else if (st.size == 8) { memcpy(&iv, s, 8); }
                else throw Error("h5lite: unsupported integer size");
                fv = (double)iv;
            }
            uint8_t* d = dst + i * dt.size;
            if (dt.cls == TypeClass::Float) {
                if (dt.size == 4) { float x = (float)fv; memcpy(d, &x, 4); }
                else { memcpy(d, &fv, 8); }
            } else {
                if (dt.size == 4) { int32_t x = (int32_t)iv; memcpy(d, &x, 4); }
                else { memcpy(d, &iv, 8); }
            }
        }
    }

    int64_t attr_int(const ObjectInfo& o, const std::string& name) {
        auto it = o.attrs.find(name);
        if (it == o.attrs.end()) throw Error("h5lite: attribute '" + name + "' not found");
        if (it->second.space.count() < 1) throw Error("h5lite: attribute '" + name + "' is empty");
        int64_t v = 0;
        convert(it->second.data.data(), it->second.type, (uint8_t*)&v, DType::i64(), 1);
        return v;
    }

    // All elements of an integer (or float) attribute, converted to int64.
    std::vector<int64_t> attr_ints(const ObjectInfo& o, const std::string& name) {
        auto it = o.attrs.find(name);
        if (it == o.attrs.end()) throw Error("h5lite: attribute '" + name + "' not found");
        uint64_t count = it->second.space.count();
        std::vector<int64_t> v((size_t)count, 0);
        if (count > 0) convert(it->second.data.data(), it->second.type, (uint8_t*)v.data(), DType::i64(), count);
        return v;
    }

  private:
    std::string path_;
    FILE* f_ = nullptr;
    uint64_t file_size_ = 0, base_ = 0, root_addr_ = 0;
    int so_ = 8, sl_ = 8;  // size of offsets / lengths

    void rd(uint64_t at, void* p, size_t n) {
        if (n == 0) return;
        if (at == kUndef || at + base_ + n > file_size_) throw Error("h5lite: read past the end of " + path_);
        if (fseeko(f_, (off_t)(at + base_), SEEK_SET) != 0 || fread(p, 1, n, f_) != n)
            throw Error("h5lite: read failed in " + path_);
    }
    std::vector<uint8_t> rdv(uint64_t at, size_t n) {
        std::vector<uint8_t> b(n);
        rd(at, b.data(), n);
        return b;
    }
    static uint64_t le(const uint8_t* p, int n) {
        uint64_t v = 0;
        for (int i = 0; i < n; i++) v |= (uint64_t)p[i] << (8 * i);
        if (n < 8 && v == ((1ull << (8 * n)) - 1)) return kUndef;  // undefined address of a narrower width
        return v;
    }
    static uint64_t lev(const uint8_t* p, int n) {  // plain value, no "undefined" widening
        uint64_t v = 0;
        for (int i = 0; i < n; i++) v |= (uint64_t)p[i] << (8 * i);
        return v;
    }

    void raw(const ObjectInfo& o, uint64_t offset, void* dst, size_t n) {
        if (o.layout_class == 0) {
            if (offset + n > o.compact.size()) throw Error("h5lite: compact dataset shorter than its dataspace");
            memcpy(dst, o.compact.data() + offset, n);
        } else {
            if (o.data_addr == kUndef) { memset(dst, 0, n); return; }  // never written: fill value
            if (offset + n > o.data_size) throw Error("h5lite: dataset storage shorter than its dataspace");
            rd(o.data_addr + offset, dst, n);
        }
    }

    void read_superblock() {
        static const uint8_t sig[8] = {0x89, 'H', 'D', 'F', '\r', '\n', 0x1a, '\n'};
        uint64_t at = 0;
        bool found = false;
        for (int tries = 0; tries < 24 && at + 8 <= file_size_; tries++) {
            uint8_t s[8];
            fseeko(f_, (off_t)at, SEEK_SET);
            if (fread(s, 1, 8, f_) == 8 && memcmp(s, sig, 8) == 0) { found = true; break; }
            at = at ? at * 2 : 512;
        }
        if (!found) throw Error("h5lite: " + path_ + " is not an HDF5 file");
        base_ = 0;
        uint8_t ver;
        rd(at + 8, &ver, 1);
        if (ver == 0 || ver == 1) {
            std::vector<uint8_t> b = rdv(at, ver == 0 ? 24 : 28);
            so_ = b[13];
            sl_ = b[14];
            if ((so_ != 8 && so_ != 4) || (sl_ != 8 && sl_ != 4)) throw Error("h5lite: unsupported offset size");
            size_t p = ver == 0 ? 24 : 28;
            std::vector<uint8_t> a = rdv(at + p, (size_t)(4 * so_ + 2 * so_ + 8 + 16));
            base_ = le(a.data(), so_);
            if (base_ == kUndef) base_ = 0;
            // root group symbol table entry follows the four addresses
            const uint8_t* e = a.data() + 4 * so_;
            root_addr_ = le(e + so_, so_);
            base_ += 0;
            if (at != 0 && base_ == 0) base_ = at;  // user block in front of the superblock
        } else if (ver == 2 || ver == 3) {
            std::vector<uint8_t> b = rdv(at, 12);
            so_ = b[9];
            sl_ = b[10];
            if (so_ != 8 || sl_ != 8) throw Error("h5lite: unsupported offset size");
            std::vector<uint8_t> a = rdv(at + 12, 32);
            base_ = le(a.data(), 8);
            if (base_ == kUndef) base_ = 0;
            root_addr_ = le(a.data() + 24, 8);
            if (at != 0 && base_ == 0) base_ = at;
        } else {
            throw Error("h5lite: unsupported superblock version");
        }
    }

    // ---- message decoding ------------------------------------------------------
    static DType dec_dtype(const uint8_t* p, size_t n) {
        if (n < 8) throw Error("h5lite: short datatype message");
        int cls = p[0] & 0x0f;
        DType t;
        t.size = (int)lev(p + 4, 4);
        t.big_endian = p[1] & 1;
        if (cls == 0) { t.cls = TypeClass::Int; t.is_signed = (p[1] & 0x08) != 0; }
        else if (cls == 1) { t.cls = TypeClass::Float; }
        else t.cls = TypeClass::Other;  // strings, compounds, ...: carried, never converted
        return t;
    }

    Dataspace dec_dspace(const uint8_t* p, size_t n) {
        if (n < 4) throw Error("h5lite: short dataspace message");
        Dataspace s;
        int ver = p[0], rank = p[1];
        size_t off;
        if (ver == 1) off = 8;
        else if (ver == 2) { off = 4; if (p[3] == 2) return s; /* null dataspace */ }
        else throw Error("h5lite: unsupported dataspace version");
        if (n < off + (size_t)rank * sl_) throw Error("h5lite: short dataspace message");
        for (int i = 0; i < rank; i++) s.dims.push_back(lev(p + off + (size_t)i * sl_, sl_));
        return s;
    }

    void dec_layout(const uint8_t* p, size_t n, ObjectInfo& o) {
        if (n < 2) throw Error("h5lite: short layout message");
        int ver = p[0];
        if (ver == 3 || ver == 4) {
            o.layout_class = p[1];
            if (o.layout_class == 1) {
                o.data_addr = le(p + 2, so_);
                o.data_size = lev(p + 2 + so_, sl_);
            } else if (o.layout_class == 0) {
                size_t sz = (size_t)lev(p + 2, 2);
                if (n < 4 + sz) throw Error("h5lite: short compact layout");
                o.compact.assign(p + 4, p + 4 + sz);
            }
        } else if (ver == 1 || ver == 2) {
            int rank = p[1];
            o.layout_class = p[2];
            size_t off = 8;
            if (o.layout_class != 0) { o.data_addr = le(p + off, so_); off += so_; }
            uint64_t sz = 1;
            for (int i = 0; i < rank; i++) { sz *= lev(p + off, 4); off += 4; }
            if (o.layout_class == 1) o.data_size = sz;  // dims here are in bytes for the last one
            if (o.layout_class == 0) {
                size_t csz = (size_t)lev(p + off, 4);
                o.compact.assign(p + off + 4, p + off + 4 + csz);
            }
            if (o.layout_class == 1) o.data_size = kUndef - 1;  // trust the dataspace
        } else {
            throw Error("h5lite: unsupported data layout version");
        }
        o.has_layout = true;
    }

    void dec_attr(const uint8_t* p, size_t n, ObjectInfo& o) {
        if (n < 8) throw Error("h5lite: short attribute message");
        int ver = p[0];
        size_t name_sz = (size_t)lev(p + 2, 2), dt_sz = (size_t)lev(p + 4, 2), ds_sz = (size_t)lev(p + 6, 2);
        size_t off = 8;
        if (ver == 3) off = 9;  // + name character set
        auto adv = [&](size_t sz) { return ver == 1 ? ((sz + 7) & ~(size_t)7) : sz; };
        if (ver != 1 && ver != 2 && ver != 3) throw Error("h5lite: unsupported attribute version");
        if ((ver == 2 || ver == 3) && (p[1] & 3)) throw Error("h5lite: shared attribute datatypes are not supported");
        if (n < off + adv(name_sz) + adv(dt_sz) + adv(ds_sz)) throw Error("h5lite: short attribute message");
        std::string name((const char*)p + off, name_sz ? name_sz - 1 : 0);
        name = name.c_str();
        off += adv(name_sz);
        AttrInfo a;
        a.type = dec_dtype(p + off, dt_sz);
        off += adv(dt_sz);
        a.space = dec_dspace(p + off, ds_sz);
        off += adv(ds_sz);
        size_t bytes = (size_t)(a.space.count() * a.type.size);
        if (n < off + bytes) throw Error("h5lite: short attribute data");
        a.data.assign(p + off, p + off + bytes);
        o.attrs[name] = a;
    }

    void dec_link(const uint8_t* p, size_t n, ObjectInfo& o) {
        if (n < 4 || p[0] != 1) throw Error("h5lite: unsupported link message");
        int flags = p[1];
        size_t off = 2;
        int ltype = 0;
        if (flags & 0x08) ltype = p[off++];
        if (flags & 0x04) off += 8;
        if (flags & 0x10) off += 1;
        int lsz = 1 << (flags & 3);
        uint64_t len = lev(p + off, lsz);
        off += lsz;
        std::string name((const char*)p + off, (size_t)len);
        off += (size_t)len;
        if (ltype != 0) return;  // soft / external links are ignored
        o.links[name] = le(p + off, so_);
    }

    void handle_msg(int type, const uint8_t* p, size_t n, ObjectInfo& o,
                    std::vector<std::pair<uint64_t, uint64_t>>& cont) {
        switch (type) {
            case 0x0001: o.space = dec_dspace(p, n); o.has_space = true; break;
            case 0x0002: {
                // link info: a defined fractal-heap address means dense link storage
                size_t off = 2;
                if (n >= 2 && (p[1] & 1)) off += 8;
                if (n >= off + 8 && le(p + off, so_) != kUndef) o.has_link_info_dense = true;
                o.is_group = true;
                break;
            }
            case 0x0003: o.type = dec_dtype(p, n); o.has_type = true; break;
            case 0x0006: dec_link(p, n, o); break;
            case 0x0008: dec_layout(p, n, o); break;
            case 0x000B: o.filtered = true; break;
            case 0x000C: dec_attr(p, n, o); break;
            case 0x0010: cont.push_back({le(p, so_), lev(p + so_, sl_)}); break;
            case 0x0011: o.btree_addr = le(p, so_); o.heap_addr = le(p + so_, so_); break;
            default: break;
        }
    }

    void parse_v1_header(uint64_t addr, ObjectInfo& o) {
        std::vector<uint8_t> pre = rdv(addr, 16);
        if (pre[0] != 1) throw Error("h5lite: unsupported object header version");
        int nmsg = (int)lev(pre.data() + 2, 2);
        uint64_t chunk_size = lev(pre.data() + 8, 4);
        std::vector<std::pair<uint64_t, uint64_t>> chunks = {{addr + 16, chunk_size}};
        int seen = 0;
        for (size_t ci = 0; ci < chunks.size() && ci < 64; ci++) {
            std::vector<uint8_t> b = rdv(chunks[ci].first, (size_t)chunks[ci].second);
            size_t off = 0;
            while (off + 8 <= b.size() && seen < nmsg) {
                int type = (int)lev(b.data() + off, 2);
                size_t sz = (size_t)lev(b.data() + off + 2, 2);
                int flags = b[off + 4];
                off += 8;
                if (off + sz > b.size()) throw Error("h5lite: object header message overruns its chunk");
                if (flags & 0x02) {
                    if (type == 0x0003 || type == 0x000B || type == 0x0001)
                        throw Error("h5lite: shared header messages are not supported");
                } else {
                    handle_msg(type, b.data() + off, sz, o, chunks);
                }
                off += sz;
                seen++;
            }
        }
    }

    void parse_v2_header(uint64_t addr, ObjectInfo& o) {
        std::vector<uint8_t> pre = rdv(addr, 6);
        if (pre[4] != 2) throw Error("h5lite: unsupported object header version");
        int flags = pre[5];
        size_t off = 6;
        if (flags & 0x20) off += 16;
        if (flags & 0x10) off += 4;
        int csz_bytes = 1 << (flags & 3);
        std::vector<uint8_t> szb = rdv(addr + off, (size_t)csz_bytes);
        uint64_t chunk0 = lev(szb.data(), csz_bytes);
        off += csz_bytes;
        const bool track_order = flags & 0x04;
        std::vector<std::pair<uint64_t, uint64_t>> chunks = {{addr + off, chunk0}};
        for (size_t ci = 0; ci < chunks.size() && ci < 64; ci++) {
            uint64_t cstart = chunks[ci].first, clen = chunks[ci].second;
            if (ci > 0) {  // continuation block: "OCHK" + messages + checksum
                std::vector<uint8_t> s = rdv(cstart, 4);
                if (memcmp(s.data(), "OCHK", 4) != 0) throw Error("h5lite: bad continuation block");
                cstart += 4;
                clen -= 8;
            }
            std::vector<uint8_t> b = rdv(cstart, (size_t)clen);
            size_t p = 0;
            const size_t hdr = track_order ? 6 : 4;
            while (p + hdr <= b.size()) {
                int type = b[p];
                size_t sz = (size_t)lev(b.data() + p + 1, 2);
                int mflags = b[p + 3];
                p += hdr;
                if (p + sz > b.size()) break;  // gap before the checksum
                if (!(mflags & 0x02)) handle_msg(type, b.data() + p, sz, o, chunks);
                p += sz;
            }
        }
    }

    // ---- old-style group lookup -------------------------------------------------
    std::string heap_string(uint64_t heap_addr, uint64_t offset) {
        std::vector<uint8_t> h = rdv(heap_addr, (size_t)(8 + 2 * sl_ + so_));
        if (memcmp(h.data(), "HEAP", 4) != 0) throw Error("h5lite: bad local heap");
        uint64_t dsize = lev(h.data() + 8, sl_);
        uint64_t daddr = le(h.data() + 8 + 2 * sl_, so_);
        if (offset >= dsize) throw Error("h5lite: link name outside the local heap");
        size_t n = (size_t)std::min<uint64_t>(dsize - offset, 1024);
        std::vector<uint8_t> s = rdv(daddr + offset, n);
        return std::string((const char*)s.data(), strnlen((const char*)s.data(), n));
    }

    bool btree_find(uint64_t node_addr, uint64_t heap_addr, const std::string& name, uint64_t* out, int depth) {
        if (depth > 32) throw Error("h5lite: group B-tree too deep");
        std::vector<uint8_t> h = rdv(node_addr, (size_t)(8 + 2 * so_));
        if (memcmp(h.data(), "TREE", 4) != 0) throw Error("h5lite: bad group B-tree node");
        if (h[4] != 0) throw Error("h5lite: not a group B-tree");
        int level = h[5];
        int used = (int)lev(h.data() + 6, 2);
        std::vector<uint8_t> body = rdv(node_addr + 8 + 2 * so_, (size_t)(used * (sl_ + so_) + sl_));
        for (int i = 0; i < used; i++) {
            uint64_t child = le(body.data() + (size_t)i * (sl_ + so_) + sl_, so_);
            if (level > 0) {
                if (btree_find(child, heap_addr, name, out, depth + 1)) return true;
            } else {
                std::vector<uint8_t> s = rdv(child, 8);
                if (memcmp(s.data(), "SNOD", 4) != 0) throw Error("h5lite: bad symbol table node");
                int nsym = (int)lev(s.data() + 6, 2);
                size_t esz = (size_t)(sl_ + so_ + 8 + 16);
                std::vector<uint8_t> e = rdv(child + 8, esz * nsym);
                for (int k = 0; k < nsym; k++) {
                    uint64_t noff = lev(e.data() + k * esz, sl_);
                    if (heap_string(heap_addr, noff) == name) {
                        *out = le(e.data() + k * esz + sl_, so_);
                        return true;
                    }
                }
            }
        }
        return false;
    }

    uint64_t lookup_link(const ObjectInfo& g, const std::string& name, const std::string& full) {
        auto it = g.links.find(name);
        if (it != g.links.end()) return it->second;
        if (g.btree_addr != kUndef) {
            uint64_t a = 0;
            if (btree_find(g.btree_addr, g.heap_addr, name, &a, 0)) return a;
        }
        if (g.has_link_info_dense)
            throw Error("h5lite: " + full + ": groups with dense (fractal-heap) link storage are not supported");
        throw Error("h5lite: " + full + ": no link named '" + name + "'");
    }
};

}  // namespace h5lite
