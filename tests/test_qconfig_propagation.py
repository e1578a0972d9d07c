"""One rule decides which QConfig a module gets, in prepare / prepare_qat / quantize_dynamic: the
contract lucid/test/unit/quantization/test_qconfig_propagation.py pins.  As there, the attribute
and spec cases are run through torch.ao.quantization as well and the sets of observed / swapped
modules must agree; the remaining cases cover the mapping form, bit widths, the two warnings and
the TypeErrors.  Host logic only: the kernels are replaced by the oracle-backed stand-in."""
import warnings

import pytest
import torch
from torch import nn

import lucid_b200.quantization as Q
from lucid_b200 import _backend
from lucid_b200.nn import quantized as nnq
from lucid_b200.nn.quantized import dynamic as nnqd
from lucid_b200.quantization._propagate import QConfigResolver, dynamic_qconfig
from lucid_b200.quantization._qscheme import per_channel_symmetric, qint4, qint8
from lucid_b200.quantization.observer import PerChannelMinMaxObserver

tq = torch.ao.quantization


@pytest.fixture(autouse=True)
def standin(monkeypatch):
    from tests import fake_ops

    cpu = torch.device("cpu")
    monkeypatch.setattr(_backend, "ops", lambda: fake_ops)
    monkeypatch.setattr(_backend, "on_cuda", lambda t: t.to(cpu))
    monkeypatch.setattr(_backend, "cuda_device", lambda index=None: cpu)


def build():
    """0 Linear, 1 ReLU, 2 Sequential(2.0 Linear, 2.1 Linear)."""
    return nn.Sequential(nn.Linear(64, 8), nn.ReLU(), nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 8)))


def at(model, path):
    for part in path.split("."):
        model = model[int(part)]
    return model


def place(model, setup, recipe):
    for path, on in setup.items():
        (model if path == "" else at(model, path)).qconfig = recipe if on else None


def observed(model):
    return {n for n, m in model.named_modules() if hasattr(m, "activation_post_process")}


# path -> True (the framework's default recipe) / None (exclude); "" is the root
ATTRIBUTE_CASES = {
    "root_only": {"": True},
    "none_at_depth_1_leaf": {"": True, "0": None},
    "none_at_depth_2_leaf": {"": True, "2.1": None},
    "none_container": {"": True, "2": None},
    "none_container_child_overrides": {"": True, "2": None, "2.0": True},
    "none_container_deep_child_overrides": {"": True, "2": None, "2.1": True},
    "none_root": {"": None},
    "none_root_child_overrides": {"": None, "0": True},
    "none_root_container_child_overrides": {"": None, "2": True},
    "none_root_and_container_leaf_overrides": {"": None, "2": None, "2.1": True},
    "only_a_leaf": {"2.0": True},
    "only_a_container": {"2": True},
    "several_none": {"": True, "0": None, "2.1": None},
}


@pytest.mark.parametrize("case", list(ATTRIBUTE_CASES))
def test_prepare_observes_what_torch_observes(case):
    setup = ATTRIBUTE_CASES[case]
    theirs = build()
    place(theirs, setup, tq.get_default_qconfig("qnnpack"))
    ours = build()
    place(ours, setup, Q.get_default_qconfig())
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        want = observed(tq.prepare(theirs))
        got = observed(Q.prepare(ours))
    assert got == want


@pytest.mark.parametrize("case", list(ATTRIBUTE_CASES))
def test_convert_quantizes_what_was_observed(case):
    model = build()
    place(model, ATTRIBUTE_CASES[case], Q.get_default_qconfig())
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        prepared = Q.prepare(model)
        prepared(torch.randn(4, 64))
        converted = Q.convert(prepared)
    quantized = {n for n, m in converted.named_modules() if isinstance(m, nnq.Linear)}
    assert quantized == {n for n in observed(prepared) if isinstance(at(prepared, n), nn.Linear)}


DYNAMIC_CASES = {
    "set_of_a_name": lambda cfg: {"0"},
    "set_of_a_container_name": lambda cfg: {"2"},
    "set_of_a_dotted_name": lambda cfg: {"2.1"},
    "set_of_a_type": lambda cfg: {nn.Linear},
    "set_of_a_name_and_a_type": lambda cfg: {"0", nn.Linear},
    "set_of_a_missing_name": lambda cfg: {"zz"},
    "dict_type_to_config": lambda cfg: {nn.Linear: cfg},
    "dict_type_and_name_none": lambda cfg: {nn.Linear: cfg, "0": None},
    "dict_dotted_name_none": lambda cfg: {nn.Linear: cfg, "2.1": None},
    "dict_container_none": lambda cfg: {nn.Linear: cfg, "2": None},
    "dict_only_none": lambda cfg: {"0": None},
    "dict_type_none": lambda cfg: {nn.Linear: None},
    "dict_name_to_config": lambda cfg: {"2": cfg},
}


def torch_dynamic(model):
    return {n for n, m in model.named_modules() if n and type(m).__module__.startswith("torch.ao.nn.quantized.dynamic")}


def ours_dynamic(model):
    return {n for n, m in model.named_modules() if n and isinstance(m, nnqd.Linear)}


@pytest.fixture
def qnnpack():
    prev = torch.backends.quantized.engine
    torch.backends.quantized.engine = "qnnpack"
    yield
    if prev in torch.backends.quantized.supported_engines:
        torch.backends.quantized.engine = prev


@pytest.mark.parametrize("case", list(DYNAMIC_CASES))
def test_dynamic_spec_forms_agree_with_torch(case, qnnpack):
    make = DYNAMIC_CASES[case]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        want = torch_dynamic(tq.quantize_dynamic(build(), make(tq.default_dynamic_qconfig)))
        got = ours_dynamic(Q.quantize_dynamic(build(), make(dynamic_qconfig(qint8))))
    assert got == want


@pytest.mark.parametrize("setup,type_spec", [({"2.0": None}, True), ({"2": None}, True), ({"0": True}, False)])
def test_dynamic_attribute_with_a_spec_agrees_with_torch(setup, type_spec, qnnpack):
    spec = {nn.Linear} if type_spec else {"2.1"}
    theirs, ours = build(), build()
    place(theirs, setup, tq.default_dynamic_qconfig)
    place(ours, setup, dynamic_qconfig(qint8))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        want = torch_dynamic(tq.quantize_dynamic(theirs, spec))
        got = ours_dynamic(Q.quantize_dynamic(ours, spec))
    assert got == want


# ---- the mapping form ----------------------------------------------------------------------
def test_module_name_none_excludes_one_module():
    mapping = Q.get_default_qconfig_mapping().set_module_name("2.1", None)
    assert observed(Q.prepare(build(), mapping)) == {"0", "2.0"}


def test_object_type_none_excludes_every_module_of_that_type():
    mapping = Q.get_default_qconfig_mapping().set_object_type(nn.Linear, None)
    with pytest.warns(UserWarning, match="matched no quantizable"):
        assert observed(Q.prepare(build(), mapping)) == set()


def test_a_module_attribute_wins_over_a_mapping_rule():
    model = build()
    model[0].qconfig = None
    mapping = Q.QConfigMapping().set_global(Q.get_default_qconfig())
    mapping.set_module_name("0", Q.get_default_qconfig())
    assert observed(Q.prepare(model, mapping)) == {"2.0", "2.1"}


def test_a_mapping_rule_applies_without_an_attribute():
    mapping = Q.QConfigMapping().set_module_name("2.0", Q.get_default_qconfig())
    assert observed(Q.prepare(build(), mapping)) == {"2.0"}


def test_a_bare_qconfig_argument_seeds_the_root():
    model = build()
    model[2].qconfig = None
    assert observed(Q.prepare(model, Q.get_default_qconfig())) == {"0"}


def test_no_attribute_and_no_argument_keeps_the_default_recipe():
    assert observed(Q.prepare(build())) == {"0", "2.0", "2.1"}


def test_a_malformed_qconfig_attribute_is_rejected():
    model = build()
    model[0].qconfig = "int8"
    with pytest.raises(TypeError, match=r"0\.qconfig must be a QConfig or None"):
        Q.prepare(model)


def test_a_malformed_argument_is_rejected():
    with pytest.raises(TypeError, match="QConfigMapping or None"):
        QConfigResolver.from_argument({"0": None}, Q.get_default_qconfig_mapping)


# ---- bit widths ----------------------------------------------------------------------------
def qint4_config():
    return Q.QConfig(activation=Q.get_default_qconfig().activation,
                     weight=PerChannelMinMaxObserver.with_args(ch_axis=0, qscheme=per_channel_symmetric, qdtype=qint4))


def max_code(model, path):
    return int(at(model, path).weight_int8.to(torch.int32).abs().max())


def calibrated(model, qconfig=None):
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        prepared = Q.prepare(model, qconfig)
        prepared(torch.randn(8, 64))
        return Q.convert(prepared)


def test_model_attribute_equals_the_argument():
    by_attribute = build()
    by_attribute.qconfig = qint4_config()
    assert max_code(calibrated(by_attribute), "0") <= 8
    assert max_code(calibrated(build(), qint4_config()), "0") <= 8


def test_default_recipe_uses_the_full_eight_bits():
    model = build()
    model.qconfig = Q.get_default_qconfig()
    assert max_code(calibrated(model), "0") > 8


def test_a_child_attribute_overrides_the_inherited_width():
    model = build()
    model.qconfig = Q.get_default_qconfig()
    model[2][0].qconfig = qint4_config()
    quantized = calibrated(model)
    assert max_code(quantized, "0") > 8 and max_code(quantized, "2.0") <= 8


def test_prepare_qat_follows_the_model_attribute():
    model = build()
    model.qconfig = Q.QConfig(
        activation=Q.get_default_qat_qconfig().activation,
        weight=Q.FakeQuantize.with_args(observer=PerChannelMinMaxObserver, ch_axis=0, qscheme=per_channel_symmetric,
                                        qdtype=qint4))
    model[2].qconfig = None
    prepared = Q.prepare_qat(model)
    assert prepared[0].weight_fake_quant.qdtype.bits == 4
    assert isinstance(prepared[2][0], nn.Linear) and not hasattr(prepared[2][0], "weight_fake_quant")


def test_prepare_qat_attribute_none_excludes_and_child_re_enters():
    model = build()
    model.qconfig = Q.get_default_qat_qconfig()
    model[2].qconfig = None
    model[2][1].qconfig = Q.get_default_qat_qconfig()
    prepared = Q.prepare_qat(model)
    assert {n for n, m in prepared.named_modules() if hasattr(m, "weight_fake_quant")} == {"0", "2.1"}


# ---- quantize_dynamic beyond what torch accepts -----------------------------------------------
def test_dtype_valued_dict_picks_the_bit_width_per_entry():
    quantized = Q.quantize_dynamic(build(), {"0": qint4, "2": qint8})
    assert max_code(quantized, "0") <= 8 and max_code(quantized, "2.0") > 8


def test_qconfig_valued_dict_takes_the_bit_width_from_the_recipe():
    assert max_code(Q.quantize_dynamic(build(), {nn.Linear: qint4_config()}), "2.1") <= 8


def test_dtype_argument_applies_to_set_entries():
    quantized = Q.quantize_dynamic(build(), {"0"}, dtype=qint4)
    assert max_code(quantized, "0") <= 8 and type(quantized[2][0]) is nn.Linear


def test_dtype_valued_none_skips_and_default_still_applies():
    quantized = Q.quantize_dynamic(build(), {nn.Linear: qint8, "2.0": None})
    assert type(quantized[2][0]) is nn.Linear and isinstance(quantized[2][1], nnqd.Linear)


def test_a_bare_linear():
    assert isinstance(Q.quantize_dynamic(nn.Linear(64, 4), {nn.Linear}), nnqd.Linear)
    with pytest.warns(UserWarning, match="no module of a targeted type"):
        assert type(Q.quantize_dynamic(nn.Linear(64, 4), {"0"})) is nn.Linear


def test_a_missing_name_warns_that_nothing_was_targeted():
    with pytest.warns(UserWarning, match="no module of a targeted type"):
        Q.quantize_dynamic(build(), {"zz"})


def test_a_named_module_without_a_dynamic_form_warns():
    with pytest.warns(UserWarning, match="Conv2d has no dynamically quantized form"):
        Q.quantize_dynamic(nn.Sequential(nn.Conv2d(1, 1, 1)), {"0"})


@pytest.mark.parametrize("spec,message", [
    ("0", "set of module types"),
    (nn.Linear, "set of module types"),
    ({3}, "keys must be nn.Module subclasses or module names"),
    ({int}, "keys must be nn.Module subclasses or module names"),
    ({"0": 8}, r"must be a QConfig, a QDtype or None"),
])
def test_bad_specs_are_rejected_before_anything_is_touched(spec, message):
    model = build()
    before = list(model.state_dict())
    with pytest.raises(TypeError, match=message):
        Q.quantize_dynamic(model, spec, inplace=True)
    assert list(model.state_dict()) == before and type(model[0]) is nn.Linear
