"""Arena loader from the reference's on-disk model format: `.sp-model` tensor table -> the resident
Q4B arena of a MoeEngine (replaces the MoE share of build_weights, src/backends/cuda/cuda_forward.cu:2222-2372,
and the pinned-arena + slot-cache machinery behind it).

File format (include/sp_engine/sp_model.h:97-134, little-endian, packed):
  512-byte header  : magic "SPMD", version 0.1, header_size, arch_id, arch struct (256 B), tokenizer hash,
                     vocab_size, tensor_count, tensor_table_offset (= 512), tensor_data_offset (multiple of
                     65536), file_size, created, transcoded_from, CRC-32 over bytes [0, 360)
  256-byte entries : name[80], dtype_id, n_dims, dims[8], offset_in_data (% 64 == 0), size_bytes, block_size,
                     block_count, blake3[32], xxh64(name); the table is sorted by that hash
Dtypes used here (sp_model.h:42-57): F32 = 1, FROBENIUS_SCALE_FP32 = 12, OK_Q4B = 13 (nibble-packed codes),
BLOCK_SCALE_FP16 = 14 (the "<weight>.bscale" sibling, f16 [rows][cols/32]).

Tensor names: the reference's loader lives in a part of its tree that is not present, so the name strings are
a table the caller can override. The defaults follow what the tree does show: GGUF-style "blk.<L>.<field>"
names (cuda_forward.cu:12191, 15091-15185), the field names of its layer struct (include/sp_engine/model.h:114-133)
and the "<weight>.bscale" sibling rule (sp_model.h:50-53).

The writer exists for tests and synthetic benchmarks only (no model file ships with the reference).
"""
import struct
import time
import zlib

import numpy as np

MAGIC = 0x444D5053           # "SPMD"
HEADER_SIZE, ENTRY_SIZE, DATA_ALIGN, TENSOR_ALIGN, CRC_COVER = 512, 256, 65536, 64, 360
DT_F32, DT_FROB_SCALE, DT_OK_Q4B, DT_BLOCK_SCALE_F16 = 1, 12, 13, 14
ARCH_GEMMA4_MOE = 11

# sp_moe_layer_weights field -> (name template, dtype of the payload)
DEFAULT_NAMES = {
    "router_w": "blk.{L}.ffn_gate_inp.weight", "router_scale": "blk.{L}.ffn_gate_inp.scale",
    "ffn_norm": "blk.{L}.ffn_norm.weight", "post_ffw1": "blk.{L}.post_ffw_norm_1.weight",
    "pre_ffw2": "blk.{L}.pre_ffw_norm_2.weight", "post_ffw2": "blk.{L}.post_ffw_norm_2.weight",
    "post_ffw": "blk.{L}.post_ffw_norm.weight", "dexps_scale": "blk.{L}.ffn_down_exps.scale",
    "gu_codes": "blk.{L}.ffn_gate_up_exps.weight", "gu_bs": "blk.{L}.ffn_gate_up_exps.weight.bscale",
    "dn_codes": "blk.{L}.ffn_down_exps.weight", "dn_bs": "blk.{L}.ffn_down_exps.weight.bscale",
    "sg_codes": "blk.{L}.ffn_gate.weight", "sg_bs": "blk.{L}.ffn_gate.weight.bscale",
    "su_codes": "blk.{L}.ffn_up.weight", "su_bs": "blk.{L}.ffn_up.weight.bscale",
    "sd_codes": "blk.{L}.ffn_down.weight", "sd_bs": "blk.{L}.ffn_down.weight.bscale",
}
_NP = {DT_F32: np.float32, DT_FROB_SCALE: np.float32, DT_OK_Q4B: np.uint8, DT_BLOCK_SCALE_F16: np.uint16}
_HDR = struct.Struct("<IHHIIII256s32sIIQQQQQI148s")
_ENT = struct.Struct("<80sII8QQQII32sQ40s")
assert _HDR.size == HEADER_SIZE and _ENT.size == ENTRY_SIZE


def xxh64(data, seed=0):
    """XXH64 of a byte string (the table's sort key is xxh64(name))."""
    P1, P2, P3, P4, P5 = 11400714785074694791, 14029467366897019727, 1609587929392839161, 9650029242287828579, 2870177450012600261
    M = (1 << 64) - 1
    rotl = lambda x, r: ((x << r) | (x >> (64 - r))) & M
    rnd = lambda acc, v: (rotl((acc + v * P2) & M, 31) * P1) & M
    n, i = len(data), 0
    if n >= 32:
        v = [(seed + P1 + P2) & M, (seed + P2) & M, seed & M, (seed - P1) & M]
        while i + 32 <= n:
            for k in range(4):
                v[k] = rnd(v[k], int.from_bytes(data[i + 8 * k:i + 8 * k + 8], "little"))
            i += 32
        h = (rotl(v[0], 1) + rotl(v[1], 7) + rotl(v[2], 12) + rotl(v[3], 18)) & M
        for k in range(4):
            h = ((h ^ rnd(0, v[k])) * P1 + P4) & M
    else:
        h = (seed + P5) & M
    h = (h + n) & M
    while i + 8 <= n:
        h = (rotl(h ^ rnd(0, int.from_bytes(data[i:i + 8], "little")), 27) * P1 + P4) & M
        i += 8
    if i + 4 <= n:
        h = (rotl(h ^ (int.from_bytes(data[i:i + 4], "little") * P1 & M), 23) * P2 + P3) & M
        i += 4
    while i < n:
        h = (rotl(h ^ (data[i] * P5 & M), 11) * P1) & M
        i += 1
    h ^= h >> 33; h = (h * P2) & M; h ^= h >> 29; h = (h * P3) & M; h ^= h >> 32
    return h


class SpModelError(ValueError):
    pass


class SpModelFile:
    """Read-only view of a `.sp-model` file: header fields and name -> tensor (numpy memmap views)."""

    def __init__(self, path):
        self.path = path
        self._mm = np.memmap(path, dtype=np.uint8, mode="r")
        if self._mm.size < HEADER_SIZE:
            raise SpModelError(f"{path}: shorter than the {HEADER_SIZE}-byte header")
        raw = bytes(self._mm[:HEADER_SIZE])
        (magic, vmaj, vmin, hsize, arch_id, arch_used, arch_cap, _arch, _tokh, vocab, count, t_off, d_off, fsize,
         created, _trans, crc, _res) = _HDR.unpack(raw)
        if magic != MAGIC:
            raise SpModelError(f"{path}: bad magic 0x{magic:08x} (want 'SPMD')")
        if hsize != HEADER_SIZE or t_off != HEADER_SIZE or d_off % DATA_ALIGN:
            raise SpModelError(f"{path}: header_size {hsize}, table offset {t_off}, data offset {d_off} break the layout rules")
        if zlib.crc32(raw[:CRC_COVER]) & 0xFFFFFFFF != crc:
            raise SpModelError(f"{path}: header CRC mismatch")
        if fsize != self._mm.size or t_off + count * ENTRY_SIZE > d_off:
            raise SpModelError(f"{path}: file_size / tensor table do not fit the file")
        self.version, self.arch_id, self.tensor_count, self.data_offset = (vmaj, vmin), arch_id, count, d_off
        self.entries = {}
        for k in range(count):
            e = _ENT.unpack(bytes(self._mm[t_off + k * ENTRY_SIZE:t_off + (k + 1) * ENTRY_SIZE]))
            name = e[0].split(b"\0", 1)[0].decode("utf-8")
            dims = tuple(int(v) for v in e[3:3 + e[2]])
            off, size = int(e[11]), int(e[12])
            if off % TENSOR_ALIGN or d_off + off + size > self._mm.size:
                raise SpModelError(f"{path}: tensor {name!r} lies outside the data region or is misaligned")
            self.entries[name] = dict(dtype_id=int(e[1]), dims=dims, offset=off, size=size, name_hash=int(e[16]))

    def tensor(self, name):
        """Flat numpy view of the tensor's payload in its storage dtype (no copy)."""
        e = self.entries.get(name)
        if e is None:
            raise SpModelError(f"{self.path}: tensor {name!r} is not in the table")
        if e["dtype_id"] not in _NP:
            raise SpModelError(f"{self.path}: tensor {name!r} has dtype {e['dtype_id']}, which the MoE path does not use")
        a = self._mm[self.data_offset + e["offset"]:self.data_offset + e["offset"] + e["size"]]
        return a.view(_NP[e["dtype_id"]])

    def moe_layer(self, L, cfg, names=DEFAULT_NAMES):
        """The sp_moe_layer_weights fields of layer L as numpy views, sizes checked against the geometry."""
        E, NE, FFE, FFS = cfg["E"], cfg["NE"], cfg["FFE"], cfg["FFS"]
        want = {"router_w": NE * E, "router_scale": E, "ffn_norm": E, "post_ffw1": E, "pre_ffw2": E, "post_ffw2": E, "post_ffw": E,
                "dexps_scale": NE, "gu_codes": NE * 2 * FFE * E // 2, "gu_bs": NE * 2 * FFE * (E // 32),
                "dn_codes": NE * E * FFE // 2, "dn_bs": NE * E * (FFE // 32), "sg_codes": FFS * E // 2, "sg_bs": FFS * (E // 32),
                "su_codes": FFS * E // 2, "su_bs": FFS * (E // 32), "sd_codes": E * FFS // 2, "sd_bs": E * (FFS // 32)}
        out = {}
        for field, n in want.items():
            a = self.tensor(names[field].format(L=L))
            if a.size != n:
                raise SpModelError(f"{self.path}: {names[field].format(L=L)!r} holds {a.size} elements, the geometry needs {n}")
            out[field] = a
        out["router_bias"] = None
        return out


def load_moe_arena(engine, path, cfg=None, names=DEFAULT_NAMES):
    """Uploads every layer's MoE tensors from `path` into the engine's resident arena."""
    f = SpModelFile(path)
    cfg = cfg or engine.cfg
    for L in range(engine.n_layers):
        engine.upload_layer(L, {k: (np.ascontiguousarray(v) if v is not None else None) for k, v in f.moe_layer(L, cfg, names).items()})
    return f


def write_sp_model(path, tensors, arch_id=ARCH_GEMMA4_MOE):
    """tensors: list of (name, dtype_id, dims, numpy array). Test/synthetic-data builder."""
    ents = []
    off = 0
    for name, dt, dims, arr in tensors:
        raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        ents.append((xxh64(name.encode()), name, dt, tuple(dims), off, raw))
        off = (off + raw.size + TENSOR_ALIGN - 1) // TENSOR_ALIGN * TENSOR_ALIGN
    ents.sort(key=lambda e: e[0])
    d_off = (HEADER_SIZE + len(ents) * ENTRY_SIZE + DATA_ALIGN - 1) // DATA_ALIGN * DATA_ALIGN
    fsize = d_off + off
    hdr = bytearray(_HDR.pack(MAGIC, 0, 1, HEADER_SIZE, arch_id, 0, 256, b"", b"", 0, len(ents), HEADER_SIZE, d_off, fsize,
                              int(time.time()), 0, 0, b""))
    struct.pack_into("<I", hdr, CRC_COVER, zlib.crc32(bytes(hdr[:CRC_COVER])) & 0xFFFFFFFF)
    with open(path, "wb") as f:
        f.write(hdr)
        for h, name, dt, dims, o, raw in ents:
            d8 = list(dims) + [0] * (8 - len(dims))
            f.write(_ENT.pack(name.encode(), dt, len(dims), *d8, o, raw.size, 1, raw.size, b"", h, b""))
        f.write(b"\0" * (d_off - HEADER_SIZE - len(ents) * ENTRY_SIZE))
        pos = 0
        for h, name, dt, dims, o, raw in sorted(ents, key=lambda e: e[4]):      # data in offset order
            f.write(b"\0" * (o - pos)); f.write(raw.tobytes()); pos = o + raw.size
        f.write(b"\0" * (off - pos))


def moe_layers_to_tensors(layers, cfg, names=DEFAULT_NAMES):
    """layers: list of dicts with the sp_moe_layer_weights fields (numpy). -> the tensor list write_sp_model takes,
    with the reference's GGUF-style dims (fastest dimension first)."""
    E, NE, FFE, FFS = cfg["E"], cfg["NE"], cfg["FFE"], cfg["FFS"]
    spec = {"router_w": (DT_F32, (E, NE)), "router_scale": (DT_F32, (E,)), "ffn_norm": (DT_F32, (E,)), "post_ffw1": (DT_F32, (E,)),
            "pre_ffw2": (DT_F32, (E,)), "post_ffw2": (DT_F32, (E,)), "post_ffw": (DT_F32, (E,)), "dexps_scale": (DT_FROB_SCALE, (NE,)),
            "gu_codes": (DT_OK_Q4B, (E, 2 * FFE, NE)), "gu_bs": (DT_BLOCK_SCALE_F16, (E // 32, 2 * FFE, NE)),
            "dn_codes": (DT_OK_Q4B, (FFE, E, NE)), "dn_bs": (DT_BLOCK_SCALE_F16, (FFE // 32, E, NE)),
            "sg_codes": (DT_OK_Q4B, (E, FFS)), "sg_bs": (DT_BLOCK_SCALE_F16, (E // 32, FFS)),
            "su_codes": (DT_OK_Q4B, (E, FFS)), "su_bs": (DT_BLOCK_SCALE_F16, (E // 32, FFS)),
            "sd_codes": (DT_OK_Q4B, (FFS, E)), "sd_bs": (DT_BLOCK_SCALE_F16, (FFS // 32, E))}
    out = []
    for L, layer in enumerate(layers):
        for field, (dt, dims) in spec.items():
            out.append((names[field].format(L=L), dt, dims, np.asarray(layer[field])))
    return out
