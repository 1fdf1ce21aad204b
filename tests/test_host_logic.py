"""Host-side behaviour that needs no GPU: the C ABI's symbols, pytree rules, param groups,
validation messages (the substrings the reference's tests match on), state layout, state dicts."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import flashoptim_jax_b200 as fo
from flashoptim_jax_b200 import _lib, tree, utils
from flashoptim_jax_b200.quantization import QuantizedArray

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "flashoptim_b200.h")).read()
    declared = set(re.findall(r"^(?:int|const char\*)\s+(fo_\w+)\s*\(", header, flags=re.M))
    assert declared == set(_lib.EXPORTS)
    lib = _lib.lib()
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.fo_version() == 3
    assert lib.fo_status_string(0) == b"ok"


def test_struct_sizes_match_the_header_layout():
    assert ctypes.sizeof(_lib.FoHyper) == 48
    assert ctypes.sizeof(_lib.FoLeaf) == 72
    assert ctypes.sizeof(_lib.FoStepDesc) == 112


def test_fo_step_rejects_bad_descriptors_without_touching_a_gpu():
    lib = _lib.lib()
    assert lib.fo_step(None, None) == 1
    d = _lib.FoStepDesc(struct_size=3)
    assert lib.fo_step(ctypes.byref(d), None) == 1 and b"ABI mismatch" in lib.fo_last_error()
    good = dict(struct_size=ctypes.sizeof(_lib.FoStepDesc), opt=0, param_dtype=1, grad_dtype=1, ecc_bits=8, state=0,
                group_size=32, n_leaves=1, n_hypers=1)
    for bad, msg in ((dict(opt=7), b"bad opt"), (dict(ecc_bits=4), b"ecc_bits"), (dict(param_dtype=0), b"fp32 params carry no ECC"),
                     (dict(state=2), b"only SGD"), (dict(group_size=0), b"group_size"), (dict(n_hypers=99), b"hyper sets")):
        d = _lib.FoStepDesc(**{**good, **bad})
        leaves = (_lib.FoLeaf * 1)()
        hypers = (_lib.FoHyper * 1)()
        d.leaves, d.hypers = ctypes.cast(leaves, ctypes.c_void_p), ctypes.cast(hypers, ctypes.c_void_p)
        assert lib.fo_step(ctypes.byref(d), None) != 0
        assert msg in lib.fo_last_error(), (bad, lib.fo_last_error())
    d = _lib.FoStepDesc(**{**good, "group_size": 2048})
    d.leaves, d.hypers = ctypes.cast((_lib.FoLeaf * 1)(), ctypes.c_void_p), ctypes.cast((_lib.FoHyper * 1)(), ctypes.c_void_p)
    assert lib.fo_step(ctypes.byref(d), None) == 2  # unsupported
    d = _lib.FoStepDesc(**{**good, "n_leaves": 0})
    assert lib.fo_step(ctypes.byref(d), None) == 0  # nothing to do


def test_structural_signature_distinguishes_exactly_what_treedefs_distinguish():
    """tree_leaves_and_signature is the cheap structure check of the donated-step cache: over random nestings of
    dicts, lists, tuples and None, equal (leaf count, signature) must mean equal TreeDef and the other way round."""
    import random

    rnd = random.Random(0)

    def grow(depth=0):
        r = rnd.random()
        if depth > 3 or r < 0.4:
            return 0
        if r < 0.5:
            return None
        if r < 0.7:
            return [grow(depth + 1) for _ in range(rnd.randint(0, 3))]
        if r < 0.85:
            return tuple(grow(depth + 1) for _ in range(rnd.randint(0, 3)))
        return {k: grow(depth + 1) for k in rnd.sample("abcd", rnd.randint(0, 3))}

    by_sig, by_def = {}, {}
    for _ in range(4000):
        t = grow()
        leaves, sig = tree.tree_leaves_and_signature(t)
        assert leaves == tree.tree_flatten(t)[0] == tree.tree_leaves(t)
        key, td = (len(leaves), repr(sig)), tree.tree_structure(t)
        assert by_sig.setdefault(key, td) == td
        assert by_def.setdefault(td, key) == key
    assert len(by_sig) == len(by_def) > 500
    assert tree.tree_leaves_and_signature([1, [2]])[1] != tree.tree_leaves_and_signature([[1], 2])[1]


def test_pytree_flattening_follows_jax_rules():
    t = {"b": [1, (2, 3)], "a": {"z": 4, "y": None}, "c": fo.FlashOptimizer(init=5, step=6)}
    leaves, td = tree.tree_flatten(t)
    assert leaves == [4, 1, 2, 3, 5, 6]  # dict keys sorted, None is an empty node
    paths = [p for p, _ in tree.tree_flatten_with_path(t)[0]]
    assert paths == [("a", "z"), ("b", 0), ("b", 1, 0), ("b", 1, 1), ("c", "init"), ("c", "step")]
    assert td.unflatten(leaves) == t
    assert td == tree.tree_structure(t) and td != tree.tree_structure({"a": 1})
    q = QuantizedArray(values=1, scales=2)
    assert tree.tree_leaves({"m": q}, is_leaf=lambda x: isinstance(x, QuantizedArray)) == [q]
    assert tree.tree_map(lambda a, b: a + b, {"x": 1, "y": [2]}, {"x": 10, "y": [20]}) == {"x": 11, "y": [22]}
    with pytest.raises(ValueError):
        tree.tree_map(lambda a, b: a, {"x": 1}, {"y": 1})


def test_param_group_selectors():
    path, leaf = ("head", "w"), object()
    m = utils._selector_matches
    assert m(path, leaf, "head") and m(path, leaf, "w") and not m(path, leaf, "trunk")
    assert m(path, leaf, "head/w") and not m(path, leaf, "head/x")
    assert m(path, leaf, ("head", "w")) and not m(path, leaf, ("head",))
    assert m(path, leaf, lambda p, l: p[0] == "head")
    assert utils._path_matches(path, leaf, ["trunk", "head"]) and not utils._path_matches(path, leaf, ["trunk"])
    cfg = utils._group_config_for_path(path, leaf, {"lr": 1, "wd": 2}, [{"params": "trunk", "lr": 9}, {"params": ["head"], "lr": 5},
                                                                         {"params": "w", "lr": 7}])
    assert cfg == {"lr": 5, "wd": 2}  # first match wins
    with pytest.raises(ValueError, match="must define a 'params' matcher"):
        utils._group_config_for_path(path, leaf, {}, [{"lr": 1}])


FACTORIES = ((fo.flash_adam, {}), (fo.flash_adamw, {}), (fo.flash_lion, {}), (fo.flash_sgd, {"momentum": 0.9}), (fo.flash_sgdw, {"momentum": 0.9}))


@pytest.mark.parametrize("factory,extra", FACTORIES, ids=["adam", "adamw", "lion", "sgd", "sgdw"])
def test_invalid_fused_group_size_is_rejected(factory, extra):
    # tests/test_optimizer_surface.py:185-199
    with pytest.raises(ValueError, match="group_size must divide BLOCK_SIZE"):
        factory(learning_rate=1e-3, quantize=True, master_weight_bits=None, group_size=40, fused=True, **extra)
    factory(learning_rate=1e-3, group_size=40, fused=False, **extra)  # legal when not fused


@pytest.mark.parametrize("factory,extra", FACTORIES, ids=["adam", "adamw", "lion", "sgd", "sgdw"])
def test_meaningless_master_weight_bits_is_rejected(factory, extra):
    # tests/test_optimizer_surface.py:202-218
    tx = factory(learning_rate=1e-3, master_weight_bits=32, fused=False, **extra)
    with pytest.raises(ValueError, match="has no effect"):
        tx.init({"x": torch.tensor([1.0, -2.0, 3.0])})


def test_meaningless_param_group_master_weight_bits_is_rejected():
    # tests/test_optimizer_surface.py:221-236
    params = {"trunk": {"w": torch.tensor([1.0, -2.0], dtype=torch.bfloat16)}, "head": {"w": torch.tensor([0.5, -0.75])}}
    tx = fo.flash_adamw(learning_rate=1e-3, master_weight_bits=24, fused=False,
                        param_groups=[{"params": ["head"], "master_weight_bits": 32}])
    with pytest.raises(ValueError, match=r"param_groups\[0\]\['master_weight_bits'\]=32 has no effect"):
        tx.init(params)


def test_other_validation_errors():
    with pytest.raises(ValueError, match="master_weight_bits must be one of"):
        fo.flash_adamw(master_weight_bits=16)
    with pytest.raises(ValueError, match="Nesterov momentum requires"):
        fo.flash_sgd(nesterov=True, momentum=0.0)
    with pytest.raises(ValueError, match="fused=True only supports parameter dtypes"):  # tests/test_adamw.py:205-211
        fo.flash_adamw(learning_rate=1e-3, fused=True).init({"x": torch.tensor([1, -2, 3], dtype=torch.int32)})
    with pytest.raises(ValueError, match="group_size must lie in"):
        fo.flash_adamw(group_size=4096, fused=False)


def test_state_layout_of_init():
    # tests/test_adamw.py:68-91,104-129,132-165,168-176; tests/test_sgd.py:93-100
    params = {"w": torch.zeros((65, 3), dtype=torch.bfloat16), "bn": torch.zeros(4)}
    st = fo.flash_adamw().init(params)
    assert st.count.dtype == torch.int32 and st.count.dim() == 0 and int(st.count) == 0
    assert isinstance(st.mu["w"], QuantizedArray) and isinstance(st.nu["bn"], QuantizedArray)
    assert st.mu["w"].values.dtype == torch.int8 and st.mu["w"].values.shape == (65, 3)
    assert st.nu["w"].values.dtype == torch.uint8 and st.mu["w"].scales.dtype == torch.float16
    assert st.mu["w"].scales.shape == (7,) and st.mu["bn"].scales.shape == (1,)
    assert st.ecc["w"].dtype == torch.int8 and st.ecc["w"].shape == (65, 3)
    assert st.ecc["bn"].dtype == torch.int32 and st.ecc["bn"].shape == ()
    st = fo.flash_adamw(master_weight_bits=32, quantize=False).init({"w": torch.zeros(5, dtype=torch.float16)})
    assert st.ecc["w"].dtype == torch.int16 and st.mu["w"].dtype == torch.float32 and st.nu["w"].shape == (5,)
    st = fo.flash_adamw(master_weight_bits=None).init({"w": torch.zeros(5, dtype=torch.bfloat16)})
    assert st.ecc["w"].dtype == torch.int32 and st.ecc["w"].shape == ()
    st = fo.flash_sgd(momentum=0.0).init({"w": torch.zeros(5, dtype=torch.bfloat16)})
    assert st.mu["w"].dtype == torch.int32 and st.mu["w"].shape == () and st.ecc["w"].dtype == torch.int8
    st = fo.flash_lion().init({"w": torch.zeros(40, dtype=torch.bfloat16)})
    assert set(st._fields) == {"count", "mu", "ecc"} and st.mu["w"].scales.shape == (2,)


def test_state_dict_round_trips_exactly():
    # tests/test_checkpointing.py:46-104
    params = {"w": torch.linspace(-2, 2, 64).to(torch.bfloat16), "b": torch.tensor([0.5, -0.75])}
    for factory, to_sd, from_sd in ((fo.flash_adamw, fo.flash_adamw_state_dict, fo.load_flash_adamw_state_dict),
                                    (lambda: fo.flash_sgd(momentum=0.9), fo.flash_sgd_state_dict, fo.load_flash_sgd_state_dict),
                                    (fo.flash_lion, fo.flash_lion_state_dict, fo.load_flash_lion_state_dict)):
        st = factory().init(params)
        st = st._replace(mu={"w": QuantizedArray(values=torch.randint(-127, 127, (64,), dtype=torch.int8),
                                                 scales=torch.rand(2).to(torch.float16)), "b": st.mu["b"]},
                         count=torch.tensor(7, dtype=torch.int32))
        sd = to_sd(st)
        assert set(sd["mu"]) == {"treedef", "leaves"} and sd["mu"]["leaves"][1]["kind"] == "quantized"
        back = from_sd(sd)
        assert int(back.count) == 7 and type(back) is type(st)
        for a, b in zip(tree.tree_leaves(back), tree.tree_leaves(st)):
            assert a.dtype == b.dtype and torch.equal(a, b)
    with pytest.raises(ValueError, match="Unsupported serialized state leaf kind"):
        utils._deserialize_state_leaf({"kind": "nope"})


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.NativeLibraryError, match="no CPU or eager fallback"):
        _lib.lib()


def test_step_refuses_cpu_tensors():
    params = {"w": torch.zeros(64, dtype=torch.bfloat16)}
    tx = fo.flash_adamw()
    st = tx.init(params)
    with pytest.raises(RuntimeError, match="computes on CUDA devices only"):
        tx.step(params, st, {"w": torch.zeros(64)})


def test_schedule_sees_zero_based_counts_and_scalar_helpers():
    from flashoptim_jax_b200 import _engine as eng
    import numpy as np

    calls = []

    def schedule(count):
        calls.append(int(count))
        return 1e-3

    assert utils._resolve_learning_rate(schedule, torch.tensor(0, dtype=torch.int32)) == 1e-3 and calls == [0]
    assert eng.one_minus(0.9, True) == np.float32(1) - np.float32(0.9)
    assert eng.one_minus(0.9, False) == np.float32(0.1)
    assert eng.one_minus(0.999, True) != eng.one_minus(0.999, False)
    assert eng.bias_correction(0.9, 1) == np.float32(1) - np.float32(0.9)


def test_warmup_cosine_schedule_host_formula():
    # examples/example_utils.py:94-103: linear warm-up to the peak, cosine decay to zero
    from flashoptim_jax_b200.schedules import warmup_cosine

    s = warmup_cosine(total_steps=100, warmup_steps=10, peak_lr=1e-3)
    assert s(0) == float(np.float32(np.float32(1e-3) * np.float32(1.0)) / np.float32(10))
    assert s(9) == float(np.float32(np.float32(1e-3) * np.float32(10.0)) / np.float32(10))  # the peak, at the last warm-up step
    assert s(10) == float(np.float32(np.float32(0.5e-3) * np.float32(2.0)))              # progress 0: cos = 1
    assert abs(s(55) - 0.5e-3) < 1e-9                                                    # half way: cos = 0
    assert abs(s(100)) < 1e-10 and s(1000) == s(100)                                      # clipped at the end
    assert warmup_cosine(50, 0, 2e-3)(0) == float(np.float32(np.float32(1e-3) * np.float32(2.0)))  # no warm-up: straight to the cosine
    assert all(s(t) >= s(t + 1) for t in range(10, 100))
