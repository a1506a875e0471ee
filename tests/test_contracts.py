"""The contract documents hold for the code."""
import pytest

from realizar_b200.utils import contracts as C


def test_block_layout_contract():
    assert C.check_block_layouts() == []


def test_required_tensor_contract_matches_synthetic_models():
    from realizar_b200.models.config import named_config
    from realizar_b200.models.weights import synthetic_weights
    for name in ("tiny-llama", "tiny-phi2", "tiny-qwen2"):
        cfg = named_config(name)
        w = synthetic_weights(cfg, seed=0)
        need = C.required_tensors(cfg.fused_qkv, cfg.gated_ffn, cfg.parallel_residual, cfg.num_layers)
        missing = [t for t in need if t not in w.tensors]
        assert missing == [], (name, missing)


@pytest.mark.gpu
def test_parameter_block_sizes_match_between_python_and_cuda(cuda_device):
    assert C.check_abi() == []
