"""An engine filled from a `.sp-model` file computes what an engine filled directly computes."""
import numpy as np
import pytest

import orc
from gpu_common import make_stack

pytestmark = pytest.mark.gpu


def test_arena_from_sp_model_equals_direct_upload(tmp_path):
    from kairos_engine_b200 import MoeEngine, sp_model, synth
    cfg, n_layers = orc.SMALL, 2
    eng, _ = make_stack(cfg, n_layers, seed=51, rand_norms=True, max_tokens=8)
    layers = [synth.layer_to_host(synth.make_layer(cfg, 51 + 1000 * L, rand_norms=True)) for L in range(n_layers)]
    path = str(tmp_path / "small.sp-model")
    sp_model.write_sp_model(path, sp_model.moe_layers_to_tensors(layers, cfg))
    eng2 = MoeEngine(n_layers=n_layers, max_tokens=8, **cfg)
    f = sp_model.load_moe_arena(eng2, path)
    assert f.tensor_count == 18 * n_layers
    x = np.random.default_rng(3).standard_normal((5, cfg["E"])).astype(np.float32)
    for flavour in (0, 1):
        y1, s1, _ = eng.forward(x, flavour=flavour)
        y2, s2, _ = eng2.forward(x, flavour=flavour)
        assert np.array_equal(s1, s2) and np.array_equal(y1.view(np.uint32), y2.view(np.uint32))
    eng.close(); eng2.close()


def test_library_loader_fills_the_arena_from_the_file(tmp_path):
    """sp_moe_load_sp_model (the C entry a daemon calls) against a file the Python writer produced - two
    independent implementations of the format - and against a directly uploaded engine; a router bias tensor in
    the file is picked up; broken files are refused with the reason."""
    from kairos_engine_b200 import MoeEngine, SpMoeError, sp_model, synth
    cfg, n_layers = orc.SMALL, 2
    bias = synth.zipf_bias(cfg["NE"], s=2.0, seed=2) * 6.0
    eng = MoeEngine(n_layers=n_layers, max_tokens=8, **cfg)
    layers = []
    for L in range(n_layers):
        layer = synth.make_layer(cfg, 61 + 1000 * L, rand_norms=True, bias=bias if L == 1 else None)
        eng.upload_layer(L, layer, on_device=True)
        layers.append(synth.layer_to_host(layer))
    tensors = sp_model.moe_layers_to_tensors(layers, cfg)
    tensors.append(("blk.1.ffn_gate_inp.bias", sp_model.DT_F32, (cfg["NE"],), bias.cpu().numpy()))
    path = str(tmp_path / "small.sp-model")
    sp_model.write_sp_model(path, tensors)
    eng2 = MoeEngine(n_layers=n_layers, max_tokens=8, **cfg)
    eng2.load_sp_model(path)
    x = np.random.default_rng(4).standard_normal((5, cfg["E"])).astype(np.float32)
    for flavour in (0, 1):
        y1, s1, _ = eng.forward(x, flavour=flavour)
        y2, s2, _ = eng2.forward(x, flavour=flavour)
        assert np.array_equal(s1, s2) and np.array_equal(y1.view(np.uint32), y2.view(np.uint32))
    # refusals: header CRC, a missing tensor (three layers asked of a two-layer file), another geometry
    raw = bytearray(open(path, "rb").read()); raw[20] ^= 1
    bad = str(tmp_path / "crc.sp-model"); open(bad, "wb").write(raw)
    with pytest.raises(SpMoeError, match="CRC"):
        eng2.load_sp_model(bad)
    eng3 = MoeEngine(n_layers=3, max_tokens=8, **cfg)
    with pytest.raises(SpMoeError, match="not in the table"):
        eng3.load_sp_model(path)
    eng4 = MoeEngine(n_layers=2, max_tokens=8, **dict(cfg, NE=32))
    with pytest.raises(SpMoeError, match="geometry needs"):
        eng4.load_sp_model(path)
    with pytest.raises(SpMoeError, match="cannot open"):
        eng2.load_sp_model(str(tmp_path / "absent.sp-model"))
    for e in (eng, eng2, eng3, eng4):
        e.close()
