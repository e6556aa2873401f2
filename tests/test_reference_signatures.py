"""Mechanical check of the drop-in boundary: every name this package re-exports from the reference's quantization
API takes the reference's parameters, in the reference's order, with the reference's defaults (extra trailing
keyword parameters are extensions).  Needs the reference checkout (skipped where it is not mounted); the GPU box
never has it."""
import dataclasses
import inspect
import os
import sys

import pytest

# the reference checkout: $LONGLIVE_REFERENCE, else a directory "reference" beside this repository
REF = os.environ.get("LONGLIVE_REFERENCE") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "fouroversix", "src")), reason="reference checkout not mounted")


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    from make_golden import _setup
    _setup(REF)
    import fouroversix
    import utils.quant as uq
    from fouroversix.model.config import ModelQuantizationConfig, ModuleQuantizationConfig
    from fouroversix.model.modules.linear import FourOverSixLinear
    from fouroversix.quantize.quantized_tensor import QuantizedTensor
    return dict(fouroversix=fouroversix, uq=uq, ModelQuantizationConfig=ModelQuantizationConfig,
                ModuleQuantizationConfig=ModuleQuantizationConfig, FourOverSixLinear=FourOverSixLinear, QuantizedTensor=QuantizedTensor)


def _params(fn):
    return [(p.name, p.kind, p.default if p.default is not inspect.Parameter.empty else "<required>")
            for p in inspect.signature(fn).parameters.values() if p.name != "self"]


def _same_prefix(ours, theirs, name):
    po, pt = _params(ours), _params(theirs)
    assert len(po) >= len(pt), f"{name}: fewer parameters than the reference ({[p[0] for p in po]} vs {[p[0] for p in pt]})"
    for a, b in zip(po, pt):
        assert a[0] == b[0], f"{name}: parameter {a[0]!r} where the reference has {b[0]!r}"
        assert a[1] == b[1] or {a[1], b[1]} <= {inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect.Parameter.KEYWORD_ONLY}, f"{name}.{a[0]}: kind"
        if b[2] != "<required>":
            assert str(a[2]) == str(b[2]) or a[2] == b[2], f"{name}.{a[0]}: default {a[2]!r} vs reference {b[2]!r}"
        else:
            assert a[2] == "<required>", f"{name}.{a[0]} is required in the reference"
    for extra in po[len(pt):]:
        assert extra[2] != "<required>", f"{name}: extension parameter {extra[0]!r} must be optional"


def test_functions_take_the_reference_parameters(ref):
    import longlive_b200 as L
    fo, uq = ref["fouroversix"], ref["uq"]
    _same_prefix(L.quantize_to_fp4, fo.quantize_to_fp4, "quantize_to_fp4")
    _same_prefix(L.fp4_matmul, fo.fp4_matmul, "fp4_matmul")
    _same_prefix(L.quantize_model, fo.quantize_model, "quantize_model")
    for name in ("dequantize_kv_cache", "k_smooth", "copy_quantized_into", "clone_quantized_tensor", "quantize_model_with_filter",
                 "_materialize_quantized_weights_for_inference"):
        _same_prefix(getattr(L.kv_cache, name), getattr(uq, name), name)


def test_classes_have_the_reference_fields_and_methods(ref):
    import longlive_b200 as L
    fo, uq = ref["fouroversix"], ref["uq"]
    for ours, theirs in ((L.QuantizationConfig, fo.QuantizationConfig), (L.ModuleQuantizationConfig, ref["ModuleQuantizationConfig"]),
                         (L.ModelQuantizationConfig, ref["ModelQuantizationConfig"]), (L.LongLiveQuantizationConfig, uq.LongLiveQuantizationConfig)):
        fo_fields = [(f.name, repr(f.default)) for f in dataclasses.fields(theirs)]
        our_fields = {f.name: repr(f.default) for f in dataclasses.fields(ours)}
        for fname, default in fo_fields:
            assert fname in our_fields, f"{ours.__name__} lacks the field {fname!r}"
            assert our_fields[fname].split(".")[-1] == default.split(".")[-1], f"{ours.__name__}.{fname}: default {our_fields[fname]} vs {default}"
    _same_prefix(L.QuantizedTensor.__init__, ref["QuantizedTensor"].__init__, "QuantizedTensor.__init__")
    _same_prefix(L.QuantizedTensor.dequantize, ref["QuantizedTensor"].dequantize, "QuantizedTensor.dequantize")
    for m in ("__init__", "get_quantized_parameters", "quantized_weight", "quantized_weight_transposed", "forward", "get_element_size"):
        _same_prefix(getattr(L.FourOverSixLinear, m), getattr(ref["FourOverSixLinear"], m), f"FourOverSixLinear.{m}")
    assert L.FourOverSixLinear.parameters_to_quantize.fget(object()) == ("weight",)
    for enum_name in ("DataType", "ScaleRule", "RoundStyle", "QuantizeBackend", "MatmulBackend"):
        theirs = getattr(fo, enum_name, None) or getattr(__import__("fouroversix.utils", fromlist=[enum_name]), enum_name)
        ours = getattr(L, enum_name)
        for member in theirs:
            if member.name in ours.__members__:
                assert ours[member.name].value == member.value
    rules = __import__("fouroversix.utils", fromlist=["ScaleRule"]).ScaleRule
    for r in rules:
        if r.name in L.ScaleRule.__members__:
            assert L.ScaleRule[r.name].cuda_id() == r.cuda_id()
