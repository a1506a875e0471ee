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


def test_kernel_parity_contract_against_compiler_reports():
    """Variants of one kernel family agree on registers ceiling, barriers and static shared memory, hot kernels do not spill
    (needs the resource reports of an in-tree build)."""
    from realizar_b200.utils import contracts
    try:
        bad = contracts.check_kernel_parity()
    except FileNotFoundError:
        pytest.skip("no compiler resource reports in this tree (run the in-tree build first)")
    assert bad == [], bad
    # the parser itself, on a literal report
    rep = ("ptxas info    : Compiling entry function '_ZN3rlz9my_kernelILi1EEEvPf' for 'sm_100a'\n"
           "ptxas info    : Function properties for _ZN3rlz9my_kernelILi1EEEvPf\n"
           "    8 bytes stack frame, 4 bytes spill stores, 12 bytes spill loads\n"
           "ptxas info    : Used 40 registers, used 1 barriers, 8 bytes cumulative stack size, 160 bytes smem\n")
    e = contracts.parse_ptxas_report(rep)
    assert e == [{"name": "_ZN3rlz9my_kernelILi1EEEvPf", "kernel": "my_kernel", "stack": 8, "spill_stores": 4, "spill_loads": 12,
                  "registers": 40, "barriers": 1, "static_smem": 160}]
