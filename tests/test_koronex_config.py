"""Koronex on the host: the configuration reader, the spec it makes, the tensors it expects, and the
planner that cuts long segments into chunks.  No GPU."""
import copy

import numpy as np
import pytest

from mini_hisparse_b200.config.koronex import KoronexConfig
from mini_hisparse_b200.config.qwen2 import ConfigError
from mini_hisparse_b200.config.registry import resolve
from mini_hisparse_b200.parts.base import Segment
from mini_hisparse_b200.parts.lightning import ChunkPlanner
from mini_hisparse_b200.weights.expected import expected_tensors_of_spec


def config():
    att = dict(heads=4, kv_heads=2, dim=16, vdim=24, mask=dict(size=10), rot=dict(dims=8, base=100.0), scale=0.5)
    return dict(architecture="Koronex", vocab=50, width=32, embedding=dict(scale=2.0), norm=dict(eps=1e-5),
                postln_alpha=1.5, token_side=dict(dim=4), layers=[
                    dict(type="attention", mixer=att, mlp=dict(kind="dense", ff=48)),
                    dict(type="lightning", mixer=dict(heads=2, dim=8, vdim=12, decay=[0.5, 0.9]), mlp=None),
                    dict(type="attention", mixer=dict(att, kv_from=0, mask=dict(size=30)), mlp=None)])


def test_spec_order_names_and_cache_needs():
    cfg, spec = resolve(config())
    assert isinstance(cfg, KoronexConfig) and cfg.alpha == 1.5 and cfg.side_dim == 4
    assert [(e.layer, e.cache_of) for e in spec.order] == [(0, None), (1, None), (2, 0)]
    names = expected_tensors_of_spec(spec)
    assert {"embed", "side.embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q.norm", "l0.mix.k.norm",
            "l0.mix.sink", "l0.mlp.up", "l1.mix.norm", "l1.side.gate", "l2.mix.q", "l2.mix.g"} <= set(names)
    assert "l2.mix.k" not in names and "l2.mix.v" not in names and "l1.norm2" not in names
    assert names["side.embed"].shape == (50, 3 * 4) and names["l0.mix.g"].shape == (4 * 24, 32)
    # the cache of layer 0 keeps the widest window among its readers; both name the same need
    from mini_hisparse_b200.parts.registry import MIXERS

    a, b = (MIXERS.build(spec.layers[i].part("mixer")) for i in (0, 2))
    assert a.cache_need() == b.cache_need() and a.cache_need().window == 30 and (a.window, b.window) == (10, 30)
    assert a.cache_need().page_shape(8) == (2 * 8 * (16 + 24),)
    assert a.plan_key() != b.plan_key()


def test_what_the_reader_refuses():
    for change in (lambda c: c.update(extra=1), lambda c: c["layers"][0]["mixer"].update(bias=True),
                   lambda c: c["layers"][0].update(type="conv"), lambda c: c["layers"][0]["mlp"].update(kind="routed"),
                   lambda c: c["layers"][2]["mixer"].update(kv_from=1), lambda c: c["layers"][2]["mixer"].update(kv_from=2),
                   lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), lambda c: c.pop("postln_alpha"),
                   lambda c: c["layers"][2]["mixer"].update(vdim=8), lambda c: c["norm"].update(kind="layer")):
        c = copy.deepcopy(config())
        change(c)
        with pytest.raises(ConfigError):
            KoronexConfig.from_dict(c)
    c = copy.deepcopy(config())
    del c["token_side"]                     # no per-layer token input: no table, no side tensors
    _, spec = resolve(c)
    assert not spec.shared and not any(n.startswith("side") or ".side." in n for n in expected_tensors_of_spec(spec))


def test_chunk_planner_cuts_long_segments_only():
    planner = ChunkPlanner(32)
    segs = [Segment("a", 0, 5, 70, 0), Segment("b", 1, 9, 1, 70), Segment("c", 2, 0, 16, 71), Segment("d", 3, 0, 17, 87)]
    arrays, facts = planner.plan(segs, 104)
    assert facts == {"num_chunks": 4, "num_long": 2}
    assert arrays["chunks"].reshape(-1, 4).tolist() == [[0, 0, 32, 0], [0, 32, 32, 1], [0, 64, 6, 2], [3, 87, 17, 0]]
    assert arrays["seg_chunks"].reshape(-1, 4).tolist() == [[0, 0, 3, 0], [3, 3, 1, 87]]
    caps = planner.capacity(104, 4)
    assert caps["chunks"] >= arrays["chunks"].size and caps["seg_chunks"] >= arrays["seg_chunks"].size
    arrays, facts = planner.plan_decode(np.asarray([3, 4]), planner.decode_fixed(2, 64))
    assert facts == {"num_chunks": 0, "num_long": 0} and arrays["chunks"].size == 0
