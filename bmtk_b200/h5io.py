"""Minimal HDF5 reader/writer for SONATA files, in pure Python + numpy.

The reference reads and writes its nodes / edges / spikes / report files with h5py
(bmtk/utils/sonata/*.py, bmtk/utils/reports/**). h5py and libhdf5 are not available where this
engine is built and run, so this module implements the subset of the HDF5 file format those files
use, behind an h5py-shaped API (File, Group, Dataset, .attrs, [] indexing). When h5py is
importable, `File` is h5py.File and nothing below is used.

Read support (what HDF5 1.8/1.10 with default settings writes, which is what every .h5 file of the
reference tree contains): superblock versions 0 and 1, version-1 object headers with continuation
blocks, old-style groups (symbol table + v1 B-tree + local heap), contiguous, compact and chunked
(v1 B-tree) dataset layouts, deflate and shuffle filters, fixed-point / floating-point / fixed and
variable-length string / enum / compound datatypes, version 1-3 attribute messages, global heap.
Write support: superblock 0, old-style groups, contiguous datasets (optionally one-chunk deflate),
numeric and string attributes (variable-length UTF-8 strings like h5py writes for `str`).
"""
import struct
import zlib

import numpy as np

try:  # pragma: no cover - not available in the build container
    import h5py as _h5py
    HAVE_H5PY = True
except ImportError:
    _h5py = None
    HAVE_H5PY = False

SIGNATURE = b'\x89HDF\r\n\x1a\n'
UNDEF = 0xFFFFFFFFFFFFFFFF


class H5Error(IOError):
    pass


# =============================================================================================
# Reader
# =============================================================================================
class _Reader(object):
    def __init__(self, path):
        with open(path, 'rb') as f:
            self.buf = f.read()
        self.path = path
        b = self.buf
        if b[:8] != SIGNATURE:
            raise H5Error('%s: not an HDF5 file' % path)
        ver = b[8]
        if ver not in (0, 1):
            raise H5Error('%s: superblock version %d is not supported (only 0 and 1)' % (path, ver))
        self.O, self.L = b[13], b[14]
        if self.O != 8 or self.L != 8:
            raise H5Error('%s: only 8-byte offsets and lengths are supported' % path)
        pos = 24 if ver == 0 else 28
        self.base, _free, self.eof, _drv = struct.unpack_from('<4Q', b, pos)
        pos += 32
        # root group symbol table entry
        _name_off, self.root_addr, cache_type = struct.unpack_from('<QQI', b, pos)
        self._gheap = {}

    # ---- primitives
    def u(self, off, n):
        return int.from_bytes(self.buf[off:off + n], 'little')

    def object_header(self, addr):
        """-> list of (type, flags, payload bytes) of a version-1 object header."""
        b = self.buf
        addr += self.base
        if b[addr:addr + 4] == b'OHDR':
            raise H5Error('%s: version-2 object headers are not supported' % self.path)
        ver = b[addr]
        if ver != 1:
            raise H5Error('%s: object header version %d at %d' % (self.path, ver, addr))
        n_msgs = self.u(addr + 2, 2)
        hdr_size = self.u(addr + 8, 4)
        msgs = []
        blocks = [(addr + 16, hdr_size)]
        while blocks and len(msgs) < n_msgs:
            pos, size = blocks.pop(0)
            end = pos + size
            while pos + 8 <= end and len(msgs) < n_msgs:
                mtype, msize, mflags = struct.unpack_from('<HHB', b, pos)
                data = b[pos + 8:pos + 8 + msize]
                pos += 8 + msize
                if mtype == 0x0010:
                    coff, clen = struct.unpack_from('<QQ', data, 0)
                    blocks.append((coff + self.base, clen))
                msgs.append((mtype, mflags, data))
        return msgs

    def local_heap_data(self, addr):
        b = self.buf
        addr += self.base
        if b[addr:addr + 4] != b'HEAP':
            raise H5Error('bad local heap at %d' % addr)
        size, _free, data_addr = struct.unpack_from('<QQQ', b, addr + 8)
        return data_addr + self.base, size

    def group_entries(self, btree_addr, heap_addr):
        """-> ordered list of (name, object header address) of an old-style group."""
        heap_data, _ = self.local_heap_data(heap_addr)
        out = []
        self._walk_group_btree(btree_addr, heap_data, out)
        return out

    def _walk_group_btree(self, addr, heap_data, out):
        b = self.buf
        addr += self.base
        if b[addr:addr + 4] != b'TREE':
            raise H5Error('bad B-tree node at %d' % addr)
        level, used = b[addr + 5], self.u(addr + 6, 2)
        pos = addr + 8 + 16
        for i in range(used):
            pos += 8  # key
            child = self.u(pos, 8)
            pos += 8
            if level > 0:
                self._walk_group_btree(child, heap_data, out)
            else:
                self._read_snod(child, heap_data, out)

    def _read_snod(self, addr, heap_data, out):
        b = self.buf
        addr += self.base
        if b[addr:addr + 4] != b'SNOD':
            raise H5Error('bad symbol table node at %d' % addr)
        n = self.u(addr + 6, 2)
        pos = addr + 8
        for _ in range(n):
            name_off, obj = struct.unpack_from('<QQ', b, pos)
            s = heap_data + name_off
            e = b.index(b'\x00', s)
            out.append((b[s:e].decode('utf-8'), obj))
            pos += 40

    def global_heap_object(self, coll_addr, index):
        if coll_addr not in self._gheap:
            b = self.buf
            a = coll_addr + self.base
            if b[a:a + 4] != b'GCOL':
                raise H5Error('bad global heap collection at %d' % a)
            size = self.u(a + 8, 8)
            objs = {}
            pos, end = a + 16, a + size
            while pos + 16 <= end:
                idx, _rc = struct.unpack_from('<HH', b, pos)
                osize = self.u(pos + 8, 8)
                if idx == 0:
                    break
                objs[idx] = b[pos + 16:pos + 16 + osize]
                pos += 16 + (osize + 7) // 8 * 8
            self._gheap[coll_addr] = objs
        return self._gheap[coll_addr].get(index, b'')

    # ---- messages
    def parse_dataspace(self, d):
        ver, rank, flags = d[0], d[1], d[2]
        if ver == 1:
            pos = 8
        elif ver == 2:
            if d[3] == 2:      # null dataspace
                return None
            pos = 4
        else:
            raise H5Error('dataspace version %d' % ver)
        return tuple(int.from_bytes(d[pos + 8 * i:pos + 8 * i + 8], 'little') for i in range(rank))

    def parse_datatype(self, d, pos=0):
        """-> (descriptor, bytes consumed). descriptor: dict(kind, dtype, size, ...)."""
        cv = d[pos]
        cls, ver = cv & 0x0F, cv >> 4
        bits = d[pos + 1] | (d[pos + 2] << 8) | (d[pos + 3] << 16)
        size = int.from_bytes(d[pos + 4:pos + 8], 'little')
        p = pos + 8
        if cls == 0:    # fixed point
            order = '>' if bits & 1 else '<'
            signed = bool(bits & 8)
            return dict(kind='int', size=size, dtype=np.dtype('%s%s%d' % (order, 'i' if signed else 'u', size))), p + 4 - pos
        if cls == 1:    # floating point
            order = '>' if bits & 1 else '<'
            return dict(kind='float', size=size, dtype=np.dtype('%sf%d' % (order, size))), p + 12 - pos
        if cls == 3:    # fixed-length string
            return dict(kind='string', size=size, dtype=np.dtype('S%d' % size), pad=bits & 0x0F,
                        utf8=((bits >> 4) & 0x0F) == 1), p - pos
        if cls == 9:    # variable length
            base, used = self.parse_datatype(d, p)
            is_str = (bits & 0x0F) == 1
            return dict(kind='vlen_str' if is_str else 'vlen', size=size, dtype=np.dtype('O'), base=base,
                        utf8=((bits >> 8) & 0x0F) == 1), p + used - pos
        if cls == 8:    # enumeration (h5py stores bool this way)
            base, used = self.parse_datatype(d, p)
            n = bits & 0xFFFF
            q = p + used
            names = []
            for _ in range(n):
                e = d.index(b'\x00', q)
                names.append(d[q:e].decode())
                if ver < 3:
                    q += (e - q + 8) // 8 * 8
                else:
                    q = e + 1
            vals = np.frombuffer(d[q:q + n * base['size']], dtype=base['dtype'])
            q += n * base['size']
            desc = dict(base)
            desc['enum'] = dict(zip(names, vals.tolist()))
            if set(names) == {'FALSE', 'TRUE'}:
                desc['kind'] = 'bool'
            return desc, q - pos
        if cls == 6:    # compound
            n = bits & 0xFFFF
            q = p
            fields = []
            for _ in range(n):
                e = d.index(b'\x00', q)
                name = d[q:e].decode()
                if ver < 3:
                    q += (e - q + 8) // 8 * 8
                    off = int.from_bytes(d[q:q + 4], 'little')
                    q += 4
                    if ver == 1:
                        q += 1 + 3 + 4 + 4 + 16
                else:
                    q = e + 1
                    nb = max(1, (size.bit_length() + 7) // 8)
                    off = int.from_bytes(d[q:q + nb], 'little')
                    q += nb
                sub, used = self.parse_datatype(d, q)
                q += used
                fields.append((name, sub['dtype'], off))
            dt = np.dtype(dict(names=[f[0] for f in fields], formats=[f[1] for f in fields],
                               offsets=[f[2] for f in fields], itemsize=size))
            return dict(kind='compound', size=size, dtype=dt), q - pos
        raise H5Error('%s: datatype class %d is not supported' % (self.path, cls))

    def decode_elements(self, raw, dt, count):
        """raw bytes -> numpy array of `count` elements for datatype descriptor dt."""
        if dt['kind'] in ('vlen_str', 'vlen'):
            out = np.empty(count, dtype=object)
            for i in range(count):
                ln, addr, idx = struct.unpack_from('<IQI', raw, 16 * i)
                data = self.global_heap_object(addr, idx)[:ln * (1 if dt['kind'] == 'vlen_str' else dt['base']['size'])] \
                    if addr not in (0, UNDEF) else b''
                if dt['kind'] == 'vlen_str':
                    out[i] = data.decode('utf-8', 'replace')
                else:
                    out[i] = np.frombuffer(data, dtype=dt['base']['dtype']).copy()
            return out
        arr = np.frombuffer(raw, dtype=dt['dtype'], count=count).copy()
        if dt['kind'] == 'bool':
            arr = arr.astype(bool)
        if dt['dtype'].kind in 'iuf' and dt['dtype'].byteorder == '>':
            arr = arr.astype(dt['dtype'].newbyteorder('<'))
        return arr

    def parse_attribute(self, d):
        ver = d[0]
        name_sz, dt_sz, ds_sz = struct.unpack_from('<HHH', d, 2)
        if ver == 1:
            pos = 8
            pad = lambda n: (n + 7) // 8 * 8  # noqa: E731
        elif ver in (2, 3):
            pos = 8 if ver == 2 else 9
            pad = lambda n: n  # noqa: E731
        else:
            raise H5Error('attribute message version %d' % ver)
        name = d[pos:pos + name_sz].split(b'\x00')[0].decode('utf-8')
        pos += pad(name_sz)
        dt, _ = self.parse_datatype(d, pos)
        pos += pad(dt_sz)
        shape = self.parse_dataspace(d[pos:pos + ds_sz])
        pos += pad(ds_sz)
        if shape is None:
            return name, None
        count = int(np.prod(shape)) if shape else 1
        arr = self.decode_elements(d[pos:], dt, count)
        if dt['kind'] == 'string':
            arr = np.array([x.split(b'\x00')[0] for x in arr.tolist()], dtype=object) if count else arr
            arr = np.array([x.decode('utf-8', 'replace') if dt.get('utf8') else x for x in arr], dtype=object)
        if shape == ():
            return name, arr[0]
        return name, arr.reshape(shape)


class _Attrs(dict):
    """Attribute mapping (read side: a plain dict filled at open time)."""


class _Node(object):
    def __init__(self, reader, addr, name):
        self._r = reader
        self._addr = addr
        self.name = name
        self._msgs = reader.object_header(addr)
        self._attrs = None

    @property
    def attrs(self):
        if self._attrs is None:
            a = _Attrs()
            for t, _f, d in self._msgs:
                if t == 0x000C:
                    k, v = self._r.parse_attribute(d)
                    a[k] = v
            self._attrs = a
        return self._attrs


class RGroup(_Node):
    def __init__(self, reader, addr, name):
        super().__init__(reader, addr, name)
        self._entries = None

    def _load(self):
        if self._entries is None:
            ent = []
            for t, _f, d in self._msgs:
                if t == 0x0011:
                    bt, heap = struct.unpack_from('<QQ', d, 0)
                    ent = self._r.group_entries(bt, heap)
                elif t in (0x0002, 0x0006):
                    raise H5Error('%s: new-style (link message) groups are not supported' % self._r.path)
            self._entries = dict(ent)
            self._order = [k for k, _ in ent]
        return self._entries

    def keys(self):
        self._load()
        return list(self._order)

    def __iter__(self):
        return iter(self.keys())

    def __len__(self):
        return len(self._load())

    def __contains__(self, key):
        try:
            self[key]
            return True
        except KeyError:
            return False

    def items(self):
        return [(k, self[k]) for k in self.keys()]

    def values(self):
        return [self[k] for k in self.keys()]

    def get(self, key, default=None):
        try:
            return self[key]
        except KeyError:
            return default

    def __getitem__(self, key):
        parts = [p for p in key.split('/') if p]
        node = self if not key.startswith('/') else _open_root(self._r)
        for p in parts:
            if not isinstance(node, RGroup):
                raise KeyError(key)
            ent = node._load()
            if p not in ent:
                raise KeyError("'%s' not found in %s" % (p, node.name))
            child_name = (node.name.rstrip('/') + '/' + p)
            node = _make_node(self._r, ent[p], child_name)
        return node


class RDataset(_Node):
    def __init__(self, reader, addr, name):
        super().__init__(reader, addr, name)
        self._dt = self._shape = self._layout = None
        self._filters = []
        for t, _f, d in self._msgs:
            if t == 0x0001:
                self._shape = reader.parse_dataspace(d)
            elif t == 0x0003:
                self._dt, _ = reader.parse_datatype(d)
            elif t == 0x0008:
                self._layout = d
            elif t == 0x000B:
                self._filters = self._parse_filters(d)
        self._cache = None

    @staticmethod
    def _parse_filters(d):
        ver, n = d[0], d[1]
        pos = 8 if ver == 1 else 2
        out = []
        for _ in range(n):
            fid = int.from_bytes(d[pos:pos + 2], 'little')
            if ver == 1 or fid >= 256:
                nlen = int.from_bytes(d[pos + 2:pos + 4], 'little')
                flags, ncd = struct.unpack_from('<HH', d, pos + 4)
                pos += 8
                pos += (nlen + 7) // 8 * 8 if ver == 1 else nlen
            else:
                flags, ncd = struct.unpack_from('<HH', d, pos + 2)
                pos += 6
            cd = [int.from_bytes(d[pos + 4 * i:pos + 4 * i + 4], 'little') for i in range(ncd)]
            pos += 4 * ncd
            if ver == 1 and ncd % 2:
                pos += 4
            out.append((fid, cd))
        return out

    @property
    def shape(self):
        return self._shape if self._shape is not None else ()

    @property
    def dtype(self):
        if self._dt['kind'] == 'bool':
            return np.dtype(bool)
        return self._dt['dtype']

    @property
    def size(self):
        return int(np.prod(self.shape)) if self.shape else 1

    @property
    def ndim(self):
        return len(self.shape)

    def __len__(self):
        if not self.shape:
            raise TypeError('scalar dataset has no len()')
        return self.shape[0]

    def _unfilter(self, raw, mask):
        for k, (fid, cd) in reversed(list(enumerate(self._filters))):
            if mask & (1 << k):
                continue
            if fid == 1:
                raw = zlib.decompress(raw)
            elif fid == 2:
                esz = cd[0] if cd else self._dt['size']
                a = np.frombuffer(raw, dtype=np.uint8)
                n = len(a) // esz
                raw = a[:n * esz].reshape(esz, n).T.tobytes() + a[n * esz:].tobytes()
            elif fid == 3:      # fletcher32: checksum trails the data
                raw = raw[:-4]
            else:
                raise H5Error('%s: HDF5 filter %d is not supported' % (self._r.path, fid))
        return raw

    def _read_all(self):
        if self._cache is not None:
            return self._cache
        r, d = self._r, self._layout
        shape = self.shape
        count = self.size
        esz = self._dt['size']
        ver = d[0]
        if ver == 3:
            cls = d[1]
            if cls == 0:
                sz = int.from_bytes(d[2:4], 'little')
                raw = d[4:4 + sz]
                arr = r.decode_elements(raw, self._dt, count)
            elif cls == 1:
                addr, sz = struct.unpack_from('<QQ', d, 2)
                if addr == UNDEF or count == 0:
                    arr = self._empty(count)
                else:
                    arr = r.decode_elements(r.buf[addr + r.base:addr + r.base + count * esz], self._dt, count)
            elif cls == 2:
                ndim = d[2]
                bt = int.from_bytes(d[3:11], 'little')
                cdims = [int.from_bytes(d[11 + 4 * i:15 + 4 * i], 'little') for i in range(ndim)]
                arr = self._read_chunked(bt, cdims[:-1])
            else:
                raise H5Error('layout class %d' % cls)
        elif ver in (1, 2):
            ndim, cls = d[1], d[2]
            pos = 8
            addr = None
            if cls != 0:
                addr = int.from_bytes(d[pos:pos + 8], 'little')
                pos += 8
            dims = [int.from_bytes(d[pos + 4 * i:pos + 4 * i + 4], 'little') for i in range(ndim)]
            pos += 4 * ndim
            if cls == 0:
                sz = int.from_bytes(d[pos:pos + 4], 'little')
                arr = r.decode_elements(d[pos + 4:pos + 4 + sz], self._dt, count)
            elif cls == 1:
                arr = self._empty(count) if addr == UNDEF or count == 0 else \
                    r.decode_elements(r.buf[addr + r.base:addr + r.base + count * esz], self._dt, count)
            else:
                arr = self._read_chunked(addr, dims[:-1])
        else:
            raise H5Error('%s: data layout version %d is not supported' % (r.path, ver))
        if self._dt['kind'] == 'string':
            pass
        arr = arr.reshape(shape) if shape else arr.reshape(())
        self._cache = arr
        return arr

    def _empty(self, count):
        if self._dt['kind'] in ('vlen_str', 'vlen'):
            return np.empty(count, dtype=object)
        return np.zeros(count, dtype=self.dtype)

    def _read_chunked(self, bt_addr, cdims):
        r = self._r
        shape = self.shape
        esz = self._dt['size']
        vl = self._dt['kind'] in ('vlen_str', 'vlen')
        out = np.empty(shape, dtype=object) if vl else np.zeros(shape, dtype=self._dt['dtype'])
        if bt_addr == UNDEF or self.size == 0:
            if self._dt['kind'] == 'bool':
                return out.astype(bool)
            return out
        ndim = len(shape)
        chunks = []
        self._walk_chunk_btree(bt_addr, ndim, chunks)
        n_el = int(np.prod(cdims))
        for size, mask, offs, addr in chunks:
            raw = self._unfilter(r.buf[addr + r.base:addr + r.base + size], mask)
            blk = r.decode_elements(raw, self._dt, n_el).reshape(cdims)
            sl_out, sl_blk = [], []
            for o, c, s in zip(offs, cdims, shape):
                n = min(c, s - o)
                sl_out.append(slice(o, o + n))
                sl_blk.append(slice(0, n))
            out[tuple(sl_out)] = blk[tuple(sl_blk)]
        return out

    def _walk_chunk_btree(self, addr, ndim, chunks):
        b = self._r.buf
        addr += self._r.base
        if b[addr:addr + 4] != b'TREE':
            raise H5Error('bad chunk B-tree node at %d' % addr)
        level, used = b[addr + 5], int.from_bytes(b[addr + 6:addr + 8], 'little')
        pos = addr + 24
        key_sz = 8 + 8 * (ndim + 1)
        for _ in range(used):
            size, mask = struct.unpack_from('<II', b, pos)
            offs = [int.from_bytes(b[pos + 8 + 8 * i:pos + 16 + 8 * i], 'little') for i in range(ndim)]
            child = int.from_bytes(b[pos + key_sz:pos + key_sz + 8], 'little')
            pos += key_sz + 8
            if level > 0:
                self._walk_chunk_btree(child, ndim, chunks)
            else:
                chunks.append((size, mask, offs, child))

    def __getitem__(self, key):
        arr = self._read_all()
        if key is Ellipsis or (isinstance(key, tuple) and len(key) == 0):
            return arr.copy() if arr.shape else arr[()]
        return arr[key]

    def __array__(self, dtype=None, copy=None):
        a = self._read_all()
        return a.astype(dtype) if dtype is not None else a

    def __iter__(self):
        return iter(self._read_all())

    def asstr(self):
        return self

    @property
    def value(self):
        return self[()]


def _make_node(reader, addr, name):
    msgs = reader.object_header(addr)
    types = {t for t, _f, _d in msgs}
    if 0x0011 in types or 0x0002 in types:
        return RGroup(reader, addr, name)
    if 0x0008 in types or 0x0001 in types:
        return RDataset(reader, addr, name)
    return RGroup(reader, addr, name)


def _open_root(reader):
    return RGroup(reader, reader.root_addr, '/')


class RFile(RGroup):
    """Read-only file object: the root group plus close()/context manager."""

    def __init__(self, path):
        r = _Reader(path)
        super().__init__(r, r.root_addr, '/')
        self.filename = path
        self.mode = 'r'

    def close(self):
        pass

    def flush(self):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


# =============================================================================================
# Writer
# =============================================================================================
def _pad8(b):
    return b + b'\x00' * (-len(b) % 8)


def _dt_message(dtype, str_len=None):
    """Datatype message body for a numpy dtype (ints, floats, bool as int8, fixed strings)."""
    dtype = np.dtype(dtype)
    if dtype.kind in 'iu':
        bits = 0x08 if dtype.kind == 'i' else 0x00
        return struct.pack('<BBBBI', 0x10 | 0, bits, 0, 0, dtype.itemsize) + struct.pack('<HH', 0, 8 * dtype.itemsize)
    if dtype.kind == 'b':
        return _dt_message(np.int8)
    if dtype.kind == 'f':
        if dtype.itemsize == 4:
            props = struct.pack('<HHBBBBI', 0, 32, 23, 8, 0, 23, 127)
            b0, b1 = 0x20, 31
        elif dtype.itemsize == 8:
            props = struct.pack('<HHBBBBI', 0, 64, 52, 11, 0, 52, 1023)
            b0, b1 = 0x20, 63
        else:
            raise H5Error('float%d is not supported' % (8 * dtype.itemsize))
        return struct.pack('<BBBBI', 0x10 | 1, b0, b1, 0, dtype.itemsize) + props
    if dtype.kind == 'S':
        return struct.pack('<BBBBI', 0x10 | 3, 0x00, 0, 0, max(1, dtype.itemsize))   # null-terminated ASCII
    raise H5Error('dtype %s cannot be written' % dtype)


def _vlen_str_dt_message():
    base = struct.pack('<BBBBI', 0x10 | 0, 0, 0, 0, 1) + struct.pack('<HH', 0, 8)   # 1-byte char, as the library writes
    # class 9, type = string (1), padding null-terminate (0), charset UTF-8 (1)
    return struct.pack('<BBBBI', 0x10 | 9, 0x01, 0x01, 0, 16) + base


def _ds_message(shape):
    if shape == ():
        return struct.pack('<BBBB4x', 1, 0, 0, 0)
    body = struct.pack('<BBBB4x', 1, len(shape), 1, 0)
    body += b''.join(struct.pack('<Q', int(s)) for s in shape)
    body += b''.join(struct.pack('<Q', int(s)) for s in shape)      # max dims = dims
    return body


class _WNode(object):
    def __init__(self, file, name):
        self.file = file
        self.name = name
        self.attrs = {}


class WDataset(_WNode):
    def __init__(self, file, name, data, compression=None):
        super().__init__(file, name)
        self.data = data
        self.compression = compression

    @property
    def shape(self):
        return self.data.shape

    @property
    def dtype(self):
        return self.data.dtype

    def __len__(self):
        return self.data.shape[0]

    def __getitem__(self, key):
        return self.data[key]

    def __setitem__(self, key, value):
        self.data[key] = value


class WGroup(_WNode):
    def __init__(self, file, name):
        super().__init__(file, name)
        self.children = {}

    def create_group(self, name):
        node = self
        for p in [q for q in name.split('/') if q]:
            if p not in node.children:
                node.children[p] = WGroup(self.file, node.name.rstrip('/') + '/' + p)
            node = node.children[p]
            if not isinstance(node, WGroup):
                raise ValueError('%s is a dataset' % p)
        return node

    def require_group(self, name):
        return self.create_group(name)

    def create_dataset(self, name, shape=None, dtype=None, data=None, compression=None, maxshape=None, chunks=None,
                       **kw):
        parts = [q for q in name.split('/') if q]
        grp = self.create_group('/'.join(parts[:-1])) if len(parts) > 1 else self
        if data is None:
            if shape is None:
                raise ValueError('shape or data is required')
            shape = (shape,) if np.isscalar(shape) else tuple(shape)
            data = np.zeros(shape, dtype=dtype if dtype is not None else np.float32)
        else:
            data = np.array(data, dtype=dtype) if dtype is not None else np.array(data)
            if data.dtype.kind == 'U':
                data = np.char.encode(data, 'utf-8')
            if data.dtype.kind == 'O':
                data = np.array([str(x).encode('utf-8') for x in data.ravel()]).reshape(data.shape)
        ds = WDataset(self.file, grp.name.rstrip('/') + '/' + parts[-1], data, compression)
        grp.children[parts[-1]] = ds
        return ds

    def __getitem__(self, key):
        node = self
        for p in [q for q in key.split('/') if q]:
            node = node.children[p]
        return node

    def __contains__(self, key):
        try:
            self[key]
            return True
        except (KeyError, AttributeError):
            return False

    def __setitem__(self, key, value):
        self.create_dataset(key, data=value)

    def keys(self):
        return list(self.children.keys())

    def items(self):
        return list(self.children.items())


class WFile(WGroup):
    """Write-mode file: the tree is kept in memory and serialised on close()."""

    def __init__(self, path):
        super().__init__(self, '/')
        self.filename = path
        self.mode = 'w'
        self._closed = False

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
        return False

    def flush(self):
        pass

    def close(self):
        if not self._closed:
            self._closed = True
            _Serializer(self).write(self.filename)

    def __del__(self):
        # like h5py, a file that was never closed is still written when the object goes away (the
        # reference's write_sonata leaves its file to the garbage collector,
        # bmtk/utils/reports/spike_trains/spikes_file_writers.py:52-71)
        try:
            self.close()
        except Exception:
            pass


class _Serializer(object):
    LEAF_K = 32       # a symbol table node holds up to 2K entries
    INTERNAL_K = 16

    def __init__(self, root):
        self.root = root
        self.buf = bytearray()
        self.gheap_objs = []      # payloads of the single global heap collection
        self.gheap_fixups = []    # (position in buf) that need the collection address

    def alloc(self, data, align=8):
        self.buf.extend(b'\x00' * (-len(self.buf) % align))
        addr = len(self.buf)
        self.buf.extend(data)
        return addr

    # ---- attributes
    def attr_message(self, name, value):
        nameb = name.encode('utf-8') + b'\x00'
        if isinstance(value, (str, bytes)) or (isinstance(value, np.ndarray) and value.dtype.kind in 'UO') \
                or (isinstance(value, (list, tuple)) and value and isinstance(value[0], str)):
            vals = [value] if isinstance(value, (str, bytes)) else list(np.asarray(value, dtype=object).ravel())
            shape = () if isinstance(value, (str, bytes)) else np.asarray(value, dtype=object).shape
            dt = _vlen_str_dt_message()
            data = b''
            fix = []
            for v in vals:
                vb = v if isinstance(v, bytes) else str(v).encode('utf-8')
                self.gheap_objs.append(vb)
                fix.append(len(data) + 4)
                data += struct.pack('<IQI', len(vb), 0, len(self.gheap_objs))
        else:
            arr = np.asarray(value)
            if arr.dtype.kind == 'b':
                arr = arr.astype(np.int8)
            if arr.dtype.kind == 'S':
                dt = _dt_message(arr.dtype)
            else:
                dt = _dt_message(arr.dtype)
            shape = arr.shape
            data = np.ascontiguousarray(arr).astype(arr.dtype.newbyteorder('<')).tobytes()
            fix = []
        ds = _ds_message(tuple(shape))
        head = struct.pack('<BBHHH', 1, 0, len(nameb), len(dt), len(ds))
        body = head + _pad8(nameb) + _pad8(dt) + _pad8(ds)
        data_off = len(body)
        body += data
        return body, [data_off + f for f in fix]

    def object_header(self, messages):
        """messages: list of (type, body, fixups). Returns address."""
        blob = bytearray()
        fixups = []
        for mtype, body, fix in messages:
            pb = _pad8(body)
            blob += struct.pack('<HHB3x', mtype, len(pb), 0)
            for f in fix:
                fixups.append(16 + len(blob) + f)
            blob += pb
        hdr = struct.pack('<BBHII4x', 1, 0, len(messages), 1, len(blob))
        addr = self.alloc(hdr + bytes(blob))
        for f in fixups:
            self.gheap_fixups.append(addr + f)
        return addr

    def attr_messages(self, node):
        out = []
        for k, v in node.attrs.items():
            body, fix = self.attr_message(k, v)
            out.append((0x000C, body, fix))
        return out

    # ---- datasets
    def write_dataset(self, ds):
        arr = np.ascontiguousarray(ds.data)
        if arr.dtype.kind == 'b':
            arr = arr.astype(np.int8)
        if arr.dtype.kind in 'iuf' and arr.dtype.byteorder == '>':
            arr = arr.astype(arr.dtype.newbyteorder('<'))
        dt = _dt_message(arr.dtype)
        dsm = _ds_message(arr.shape)
        raw = arr.tobytes()
        msgs = [(0x0001, dsm, []), (0x0003, dt, [])]
        # fill value, version 2, the library's default: allocate early, write if set, defined, size 0
        msgs.append((0x0005, struct.pack('<BBBBI', 2, 2, 2, 1, 0), []))
        if ds.compression in ('gzip', 'deflate', True) and arr.size > 0 and arr.ndim >= 1:
            comp = zlib.compress(raw, 4)
            data_addr = self.alloc(comp)
            ndim = arr.ndim
            # one chunk covering the dataset: a single-entry level-0 chunk B-tree node
            key0 = struct.pack('<II', len(comp), 0) + b''.join(struct.pack('<Q', 0) for _ in range(ndim + 1))
            key1 = struct.pack('<II', 0, 0) + b''.join(struct.pack('<Q', int(s)) for s in arr.shape) + struct.pack('<Q', 0)
            node = b'TREE' + struct.pack('<BBHQQ', 1, 0, 1, UNDEF, UNDEF) + key0 + struct.pack('<Q', data_addr) + key1
            # pad the node to its full size (2K+1 keys, 2K children with K = 32, the library default)
            full = 24 + (2 * 32 + 1) * len(key0) + 2 * 32 * 8
            node += b'\x00' * (full - len(node))
            bt_addr = self.alloc(node)
            layout = struct.pack('<BBB', 3, 2, ndim + 1) + struct.pack('<Q', bt_addr)
            layout += b''.join(struct.pack('<I', int(s)) for s in arr.shape) + struct.pack('<I', arr.dtype.itemsize)
            filt = struct.pack('<BB6x', 1, 1) + struct.pack('<HHHH', 1, 8, 1, 1) + b'deflate\x00' + struct.pack('<II', 4, 0)
            msgs.append((0x000B, filt, []))
        else:
            data_addr = self.alloc(raw) if raw else UNDEF
            layout = struct.pack('<BB', 3, 1) + struct.pack('<QQ', data_addr, len(raw))
        msgs.append((0x0008, layout, []))
        msgs += self.attr_messages(ds)
        return self.object_header(msgs)

    # ---- groups
    def write_group(self, grp):
        names = sorted(grp.children.keys(), key=lambda s: s.encode('utf-8'))
        child_addr = {}
        for n in names:
            c = grp.children[n]
            child_addr[n] = self.write_group(c) if isinstance(c, WGroup) else self.write_dataset(c)
        # local heap: offset 0 holds the empty string
        heap = bytearray(b'\x00' * 8)
        offs = {}
        for n in names:
            offs[n] = len(heap)
            heap += _pad8(n.encode('utf-8') + b'\x00')
        free_off = len(heap)
        heap += struct.pack('<QQ', 1, 16)          # one free block: next = 1 (none), size 16
        heap_data = self.alloc(bytes(heap))
        heap_addr = self.alloc(b'HEAP' + struct.pack('<B3xQQQ', 0, len(heap), free_off, heap_data))
        # symbol table nodes
        per = 2 * self.LEAF_K
        snods = []
        for i in range(0, max(len(names), 1), per):
            part = names[i:i + per]
            body = b'SNOD' + struct.pack('<BBH', 1, 0, len(part))
            for n in part:
                body += struct.pack('<QQII16x', offs[n], child_addr[n], 0, 0)
            body += b'\x00' * (40 * (per - len(part)))
            snods.append((self.alloc(body), offs[part[-1]] if part else 0))
        if len(snods) > 2 * self.INTERNAL_K:
            raise H5Error('group %s has too many members for this writer' % grp.name)
        node = b'TREE' + struct.pack('<BBHQQ', 0, 0, len(snods), UNDEF, UNDEF) + struct.pack('<Q', 0)
        for addr, last_off in snods:
            node += struct.pack('<QQ', addr, last_off)
        full = 24 + (2 * self.INTERNAL_K + 1) * 8 + 2 * self.INTERNAL_K * 8
        node += b'\x00' * (full - len(node))
        bt_addr = self.alloc(node)
        msgs = [(0x0011, struct.pack('<QQ', bt_addr, heap_addr), [])] + self.attr_messages(grp)
        addr = self.object_header(msgs)
        grp._bt, grp._heap = bt_addr, heap_addr
        return addr

    def write(self, path):
        self.buf = bytearray(b'\x00' * 96)      # superblock (56 bytes + 40-byte root entry)
        root_addr = self.write_group(self.root)
        if self.gheap_objs:
            body = bytearray()
            for i, vb in enumerate(self.gheap_objs):
                body += struct.pack('<HHIQ', i + 1, 0, 0, len(vb)) + _pad8(vb)
            size = max(4096, 16 + len(body) + 16)
            free = size - 16 - len(body)
            coll = b'GCOL' + struct.pack('<B3xQ', 1, size) + bytes(body) + struct.pack('<HHIQ', 0, 0, 0, free)
            coll += b'\x00' * (size - len(coll))
            gaddr = self.alloc(coll)
            for pos in self.gheap_fixups:
                self.buf[pos:pos + 8] = struct.pack('<Q', gaddr)
        eof = len(self.buf)
        sb = SIGNATURE + struct.pack('<BBBBBBBBHHI', 0, 0, 0, 0, 0, 8, 8, 0, self.LEAF_K, self.INTERNAL_K, 0)
        sb += struct.pack('<QQQQ', 0, UNDEF, eof, UNDEF)
        sb += struct.pack('<QQII', 0, root_addr, 1, 0) + struct.pack('<QQ', self.root._bt, self.root._heap)
        self.buf[0:len(sb)] = sb
        with open(path, 'wb') as f:
            f.write(self.buf)


def File(path, mode='r', **kw):
    """h5py.File when h5py is installed, else the built-in reader ('r') or writer ('w')."""
    if HAVE_H5PY:
        return _h5py.File(path, mode, **kw)
    if mode in ('r', 'r+'):
        return RFile(path)
    if mode in ('w', 'x', 'w-'):
        return WFile(path)
    raise H5Error("mode '%s' is not supported without h5py (use 'r' or 'w')" % mode)


Group = (RGroup, WGroup) if not HAVE_H5PY else _h5py.Group
Dataset = (RDataset, WDataset) if not HAVE_H5PY else _h5py.Dataset
