"""Dotivik on the host: the configuration reader, the spec it makes (run order with repeated layers, a
cache per pass, the stream input before every pass), the tensors it expects and the caches it asks for.
No GPU."""
import copy

import pytest

from mini_hisparse_b200.config.dotivik import DotivikConfig
from mini_hisparse_b200.config.qwen2 import ConfigError
from mini_hisparse_b200.config.registry import resolve
from mini_hisparse_b200.parts.registry import MIXERS
from mini_hisparse_b200.parts.spec import PagedKVNeed, PagedRowsNeed
from mini_hisparse_b200.weights.expected import expected_tensors_of_spec


def config():
    att = dict(heads=6, kv_heads=3, dim=16, vdim=24, scale=0.3, softcap=20.0, diff=0.4, rot=dict(dims=8, base=100.0))
    lat = dict(heads=5, dim=8, rot_dim=4, vdim=12, kv_rank=20, scale=0.2, mask=dict(size=11), rot=dict(dims=4, base=50.0))
    return dict(architecture="Dotivik", vocab=50, width=40, norm=dict(eps=1e-5), loop=dict(start=1, stop=3, times=3),
                layers=[dict(type="attention", mixer=att, mlp=dict(kind="dense", ff=48)),
                        dict(type="latent_attention", mixer=lat, mlp=None),
                        dict(type="attention", mixer=att, mlp=dict(kind="dense", ff=56)),
                        dict(type="latent_attention", mixer=lat, mlp=dict(kind="dense", ff=48))])


def test_run_order_names_and_cache_needs():
    cfg, spec = resolve(config())
    assert isinstance(cfg, DotivikConfig) and cfg.loop.times == 3
    # layers 1 and 2 run three times; every pass opens with the stream input; every entry owns a cache
    assert [(e.layer, e.before) for e in spec.order] == [(0, None), (1, "loop"), (2, None), (1, "loop"), (2, None),
                                                         (1, "loop"), (2, None), (3, None)]
    assert all(e.cache_of is None for e in spec.order)
    names = expected_tensors_of_spec(spec)
    assert {"embed", "loop.in", "final.norm", "l0.norm1", "l0.mix.lq1", "l0.mix.lk2", "l0.mix.g", "l0.mlp.gate",
            "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv", "l3.mlp.down"} <= set(names)
    assert not any(n.startswith("l1.mlp") or n.endswith("norm2") for n in names)
    assert not [n for n, ps in names.items() if n.startswith("head") and not ps.optional]     # the head is the table
    assert names["loop.in"].shape == (40, 80) and names["l0.mix.q"].shape == (6 * 2 * 16, 40)
    assert names["l0.mix.k"].shape == (3 * 2 * 16, 40) and names["l0.mix.v"].shape == (3 * 24, 40)
    assert names["l0.mix.g"].shape == (6, 40) and names["l0.mix.o"].shape == (40, 6 * 24)
    assert names["l1.mix.q"].shape == (5 * 12, 40) and names["l1.mix.dkv"].shape == (24, 40)
    assert names["l1.mix.uk"].shape == (5 * 8, 20) and names["l1.mix.uv"].shape == (5 * 12, 20)
    a, b = (MIXERS.build(spec.layers[i].part("mixer")) for i in (0, 1))
    assert a.cache_need() == PagedKVNeed(kv_heads=3, head_dim=32, v_dim=24) and a.cache_need().window is None
    assert a.cache_need().page_shape(8) == (3 * 8 * (32 + 24),)
    assert b.cache_need() == PagedRowsNeed(width=24, window=11) and b.cache_need().page_shape(8) == (8, 24)


def test_without_a_loop_and_with_an_empty_one():
    for change in (lambda c: c.pop("loop"), lambda c: c.update(loop=None), lambda c: c["loop"].update(start=2, stop=2)):
        c = config()
        change(c)
        _, spec = resolve(c)
        assert [(e.layer, e.before) for e in spec.order] == [(i, None) for i in range(4)]
        assert not spec.shared and "loop.in" not in expected_tensors_of_spec(spec)
    c = config()
    c["loop"] = dict(start=0, stop=4, times=1)       # one pass over everything still opens with the stream input
    _, spec = resolve(c)
    assert [(e.layer, e.before) for e in spec.order] == [(0, "loop"), (1, None), (2, None), (3, None)]


def test_what_the_reader_refuses():
    for change in (lambda c: c.update(extra=1), lambda c: c["layers"][0]["mixer"].update(bias=True),
                   lambda c: c["layers"][0].update(type="conv"), lambda c: c["layers"][0]["mlp"].update(kind="routed"),
                   lambda c: c["layers"][0]["mixer"].update(kv_heads=4), lambda c: c["layers"][0]["mixer"].pop("diff"),
                   lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), lambda c: c["layers"][1]["mixer"].pop("kv_rank"),
                   lambda c: c["layers"][1]["mixer"]["rot"].update(dims=2), lambda c: c["layers"][1]["mixer"].update(mask=dict(size=0)),
                   lambda c: c["loop"].update(stop=5), lambda c: c["loop"].update(times=0), lambda c: c["norm"].update(kind="rms"),
                   lambda c: c.pop("width")):
        c = copy.deepcopy(config())
        change(c)
        with pytest.raises(ConfigError):
            DotivikConfig.from_dict(c)
