"""CPU tests: every demo command of the apps package runs through the CLI with tiny step counts and returns results
that show the demo did its job (reference: the ``bin/*.dart`` demo programs)."""
import math

import pytest

from dart_pytorch_b200.apps.__main__ import all_demos, main as cli

REFERENCE_DEMOS = [
    "gpt_demo", "lm_demo", "aft_demo", "aft_bench", "seq2seq_optim_bench", "word2vec_demo", "data_loaders_demo",
    "tutorial", "vit_face_recognition_demo", "vit_object_detection_demo", "vit_hungarian_matching_demo",
    "vit_hungarian_batch_demo", "train_face_folder", "multi_modal_demo", "train_multimodal_demo",
    "train_muzero_shakespeare", "train_llama_vision_demo", "train_llava_projector", "llama_llava_demo",
    "llama_image_rag", "clip_smoke", "lc0_bench_batch", "rag_learn", "rag_demo", "rag_gpu_demo", "rag_qa_demo", "qa",
    "vector_store_demo", "gpt2_hf_demo", "vector_chunked_rag_demo", "vector_cluster_demo", "vector_dedup_demo",
    "vector_image_search_demo", "vector_index_benchmark_demo", "vector_zero_shot_classify_demo", "bug_repro",
    "gpt2_debug", "prep_coco_pairs", "hello",
]


def _finite(x) -> bool:
    if isinstance(x, float):
        return math.isfinite(x)
    if isinstance(x, dict):
        return all(_finite(v) for v in x.values())
    if isinstance(x, (list, tuple)):
        return all(_finite(v) for v in x)
    return True


def test_every_reference_demo_is_registered():
    assert set(REFERENCE_DEMOS) <= set(all_demos())


@pytest.mark.parametrize("name", REFERENCE_DEMOS)
def test_demo_runs(name, capsys):
    extra = ["--n", "300"] if name == "vector_index_benchmark_demo" else []
    res = cli([name, "--device", "cpu", "--steps", "3", "--seed", "0"] + extra)
    assert isinstance(res, dict) and res and _finite(res)
    assert capsys.readouterr().out.strip()


def test_demos_learn_and_check_what_they_claim():
    res = cli(["gpt_demo", "--device", "cpu", "--steps", "40"])
    assert res["loss_last"] < 0.5 * res["loss_first"] and res["cache_equal"]
    res = cli(["tutorial", "--device", "cpu", "--steps", "200"])
    assert res["grad"] == [[2.0, 4.0], [6.0, 8.0]] and res["fit_loss"] < 0.05 and res["reload_identical"]
    res = cli(["vit_object_detection_demo", "--device", "cpu", "--steps", "60"])
    assert res["box_err_last"] < res["box_err_first"]
    res = cli(["train_llava_projector", "--device", "cpu", "--steps", "40"])
    assert res["frozen_untouched"] and res["loss_last"] < res["loss_first"] and res["trainable"] < res["total"]
    res = cli(["train_llama_vision_demo", "--device", "cpu", "--steps", "60"])
    assert res["loss_last"] < 0.5 * res["loss_first"]
    res = cli(["train_muzero_shakespeare", "--device", "cpu", "--steps", "40"])
    assert res["loss_last"] < res["loss_first"]
    res = cli(["gpt2_hf_demo", "--device", "cpu"])
    assert res["max_abs_diff"] < 1e-5 and res["loaded"] > 0
    res = cli(["llama_image_rag", "--device", "cpu"])
    assert res["top_is_source"]
    res = cli(["vector_image_search_demo", "--device", "cpu"])
    assert res["top_is_source"]
    res = cli(["vector_dedup_demo", "--device", "cpu"])
    assert [0, 9] in res["groups"]
    res = cli(["qa", "--device", "cpu"])
    assert res["reloaded"] == res["chunks"] == 10
    res = cli(["vector_index_benchmark_demo", "--device", "cpu", "--n", "400"])
    assert res["recall"]["Flat"] == 1.0 and res["recall"]["HNSW16"] > 0.9
    res = cli(["data_loaders_demo", "--device", "cpu"])
    assert res["list_batches"] == [4, 4, 2] and res["lm_shift_ok"] and res["image_classes"] == 2
    res = cli(["bug_repro", "--device", "cpu"])
    assert res["finite"] and res["nonzero"] and res["loss_last"] > 0
    res = cli(["prep_coco_pairs"])
    assert res["pairs"] == 3 and "000000000001.txt" in res["files"]
