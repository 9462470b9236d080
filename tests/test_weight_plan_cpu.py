"""The DNN layer's weight-only plan on the host: the reference's own tests of its configuration types and metadata
(crates/oxicuda-dnn/src/quantize/gptq_awq.rs:1204-1330, :1456-1525) restated; no device is needed."""
import pytest

from oxicuda_b200.dnn_weight_quant import AwqConfig, GptqConfig, QuantMethodTag, WeightQuantMethod, WeightQuantPlan
from oxicuda_b200.errors import DnnError


def test_gptq_config_validation():  # gptq_awq.rs:1207-1243
    GptqConfig(bits=4, group_size=128, block_size=128, damp_percent=0.01, symmetric=True, act_order=False, true_sequential=True).validate()
    with pytest.raises(DnnError) as e:
        GptqConfig(bits=5).validate()
    assert e.value.variant == "InvalidArgument" and "bits must be 2, 3, 4, or 8" in str(e.value)
    for bad in (GptqConfig(group_size=0), GptqConfig(block_size=0), GptqConfig(damp_percent=-0.1)):
        with pytest.raises(DnnError):
            bad.validate()
    for bits in (2, 3, 4, 8):
        GptqConfig(bits=bits).validate()


def test_awq_config_validation():  # gptq_awq.rs:1245-1277
    AwqConfig(bits=4, group_size=128, zero_point=True, search_alpha_min=0.0, search_alpha_max=1.0, search_steps=20).validate()
    with pytest.raises(DnnError):
        AwqConfig(bits=3).validate()
    with pytest.raises(DnnError) as e:
        AwqConfig(search_alpha_min=1.0, search_alpha_max=0.0).validate()
    assert "alpha_min" in str(e.value)
    for bad in (AwqConfig(group_size=0), AwqConfig(search_steps=0)):
        with pytest.raises(DnnError):
            bad.validate()


def test_quantized_weight_info():  # gptq_awq.rs:1280-1331
    info = WeightQuantPlan(WeightQuantMethod.Gptq(GptqConfig(bits=4, group_size=128, symmetric=True)), 256, 1024).quantized_weight_info()
    assert (info.bits, info.rows, info.cols) == (4, 256, 1024)
    assert info.packed_weight_elements == 32768 and info.scale_elements == 2048          # 8 codes per word; 8 groups per row
    assert not info.has_zero_point and info.zero_point_elements == 0 and info.method is QuantMethodTag.Gptq
    info = WeightQuantPlan(WeightQuantMethod.Awq(AwqConfig(bits=8, group_size=128, zero_point=True)), 128, 512).quantized_weight_info()
    assert info.bits == 8 and info.packed_weight_elements == 16384 and info.scale_elements == 512
    assert info.has_zero_point and info.zero_point_elements == 512 and info.method is QuantMethodTag.Awq
    assert WeightQuantPlan(WeightQuantMethod.Gptq(GptqConfig(bits=3)), 4, 128).elements_per_u32() == 10  # two bits of each word unused


def test_plan_scratch_and_launch_figures():  # gptq_awq.rs:1455-1505
    plan = WeightQuantPlan(WeightQuantMethod.Gptq(GptqConfig(block_size=128, act_order=True)), 256, 1024)
    assert plan.workspace_bytes() == 1024 * 4 + 1024 * 4 + 256 * 128 * 4
    assert WeightQuantPlan(WeightQuantMethod.Gptq(GptqConfig(block_size=128)), 64, 128).shared_memory_bytes() == 128 * 4
    assert WeightQuantPlan(WeightQuantMethod.Awq(AwqConfig(group_size=64)), 64, 128).shared_memory_bytes() == 64 * 4
    assert WeightQuantPlan(WeightQuantMethod.Gptq(), 512, 1024).launch_params() == (2, 256)
    assert WeightQuantPlan(WeightQuantMethod.Awq(), 4, 128).launch_params() == (2, 256)       # one thread per element


def test_plan_construction_errors():  # gptq_awq.rs:254-284, :1507-1523
    with pytest.raises(DnnError) as e:
        WeightQuantPlan(WeightQuantMethod.Gptq(GptqConfig(group_size=100)), 64, 256)
    assert e.value.variant == "InvalidArgument" and "divisible" in str(e.value)
    with pytest.raises(DnnError) as e:
        WeightQuantPlan(WeightQuantMethod.Gptq(), 0, 128)
    assert e.value.variant == "InvalidDimension"
    with pytest.raises(DnnError):
        WeightQuantPlan(WeightQuantMethod.Gptq(GptqConfig(bits=5)), 64, 128)


def test_fused_gemv_checks_its_tensors_before_any_device_work():
    class Fake:                                                          # stands in for a device tensor: only numel() is looked at
        def __init__(self, n):
            self._n = n

        def numel(self):
            return self._n

    plan = WeightQuantPlan(WeightQuantMethod.Gptq(), 64, 128)
    with pytest.raises(DnnError) as e:
        plan.fused_dequant_gemv(Fake(100), Fake(64), Fake(128))
    assert e.value.variant == "BufferTooSmall" and (e.value.expected, e.value.actual) == (64 * 16 * 4, 400)
    with pytest.raises(DnnError) as e:
        plan.fused_dequant_gemv(Fake(64 * 16), Fake(63), Fake(128))
    assert (e.value.expected, e.value.actual) == (64 * 4, 63 * 4)
    with pytest.raises(DnnError) as e:
        plan.fused_dequant_gemv(Fake(64 * 16), Fake(64), Fake(127))
    assert (e.value.expected, e.value.actual) == (128 * 4, 127 * 4)
