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
