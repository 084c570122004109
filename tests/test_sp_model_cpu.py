"""The `.sp-model` reader/writer against the layout rules of include/sp_engine/sp_model.h:97-134."""
import os
import struct
import sys
import zlib

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kairos_engine_b200 import sp_model  # noqa: E402

CFG = dict(E=64, NE=4, NU=2, FFE=32, FFS=64)


def _layer(seed):
    r = np.random.default_rng(seed)
    E, NE, FFE, FFS = CFG["E"], CFG["NE"], CFG["FFE"], CFG["FFS"]
    f32 = lambda *s: r.standard_normal(s).astype(np.float32)
    u8 = lambda n: r.integers(0, 256, n, dtype=np.uint8)
    u16 = lambda n: r.integers(0, 1 << 15, n, dtype=np.uint16)
    return dict(router_w=f32(NE, E), router_scale=f32(E), ffn_norm=f32(E), post_ffw1=f32(E), pre_ffw2=f32(E), post_ffw2=f32(E),
                post_ffw=f32(E), dexps_scale=f32(NE), gu_codes=u8(NE * 2 * FFE * E // 2), gu_bs=u16(NE * 2 * FFE * E // 32),
                dn_codes=u8(NE * E * FFE // 2), dn_bs=u16(NE * E * FFE // 32), sg_codes=u8(FFS * E // 2), sg_bs=u16(FFS * E // 32),
                su_codes=u8(FFS * E // 2), su_bs=u16(FFS * E // 32), sd_codes=u8(E * FFS // 2), sd_bs=u16(E * FFS // 32))


def test_xxh64_known_answers():
    # published XXH64 test values (seed 0)
    assert sp_model.xxh64(b"") == 0xEF46DB3751D8E999
    assert sp_model.xxh64(b"a") == 0xD24EC4F1A98C6E5B
    assert sp_model.xxh64(b"abc") == 0x44BC2CF5AD770999


def test_round_trip_and_layout_rules(tmp_path):
    layers = [_layer(1), _layer(2)]
    p = tmp_path / "tiny.sp-model"
    sp_model.write_sp_model(str(p), sp_model.moe_layers_to_tensors(layers, CFG))
    raw = p.read_bytes()
    assert raw[:4] == b"SPMD" and struct.unpack_from("<I", raw, 8)[0] == 512
    assert struct.unpack_from("<Q", raw, 328)[0] % 65536 == 0                       # data region alignment
    assert zlib.crc32(raw[:360]) & 0xFFFFFFFF == struct.unpack_from("<I", raw, 360)[0]
    f = sp_model.SpModelFile(str(p))
    assert f.arch_id == sp_model.ARCH_GEMMA4_MOE and f.tensor_count == 2 * 18
    hashes = [e["name_hash"] for e in f.entries.values()]
    assert hashes == sorted(hashes) and all(e["offset"] % 64 == 0 for e in f.entries.values())
    assert f.entries["blk.1.ffn_gate_up_exps.weight"]["dims"] == (CFG["E"], 2 * CFG["FFE"], CFG["NE"])
    for L, layer in enumerate(layers):
        got = f.moe_layer(L, CFG)
        for k, v in layer.items():
            assert np.array_equal(got[k], np.asarray(v).reshape(-1)), k


def test_errors_are_loud(tmp_path):
    p = tmp_path / "bad.sp-model"
    sp_model.write_sp_model(str(p), sp_model.moe_layers_to_tensors([_layer(3)], CFG))
    raw = bytearray(p.read_bytes())
    raw[20] ^= 1                                                                  # header byte under the CRC
    (tmp_path / "crc.sp-model").write_bytes(raw)
    with pytest.raises(sp_model.SpModelError, match="CRC"):
        sp_model.SpModelFile(str(tmp_path / "crc.sp-model"))
    f = sp_model.SpModelFile(str(p))
    with pytest.raises(sp_model.SpModelError, match="not in the table"):
        f.moe_layer(1, CFG)                                                       # only layer 0 exists
    with pytest.raises(sp_model.SpModelError, match="geometry"):
        f.moe_layer(0, dict(CFG, NE=8))
