"""GPU tests: every demo command runs with ``--device cuda`` (tiny shapes through the native kernels' small-shape
paths) and the training demos still learn there."""
import pytest

from dart_pytorch_b200.apps.__main__ import all_demos, main as cli

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", sorted(all_demos()))
def test_demo_runs_on_cuda(name, capsys):
    extra = ["--n", "300"] if name == "vector_index_benchmark_demo" else []
    res = cli([name, "--device", "cuda", "--steps", "3", "--seed", "0"] + extra)
    assert isinstance(res, dict) and res
    assert capsys.readouterr().out.strip()


def test_training_demos_learn_on_cuda():
    res = cli(["gpt_demo", "--device", "cuda", "--steps", "30"])
    assert res["loss_last"] < 0.5 * res["loss_first"] and res["cache_equal"]
    res = cli(["train_llama_vision_demo", "--device", "cuda", "--steps", "40"])
    assert res["loss_last"] < 0.7 * res["loss_first"]
    res = cli(["rag_gpu_demo", "--device", "cuda", "--steps", "2"])
    assert res["max_abs_diff"] < 1e-4
    res = cli(["gpt2_hf_demo", "--device", "cuda"])
    assert res["max_abs_diff"] < 1e-4
