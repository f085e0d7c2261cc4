"""Worker of the tensor-parallel Llama test (launched by torch.distributed.run, one rank per GPU): shards a small Llama
over the ranks and checks prefill logits, eager decode and graph-replayed decode against the whole model."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dart_pytorch_b200 import _native  # noqa: E402
from dart_pytorch_b200.models.llama import Llama, LlamaConfig  # noqa: E402
from dart_pytorch_b200.parallel.tp_llama import TPLlamaEngine  # noqa: E402


def full_logits(engine, B):
    parts = [torch.empty_like(engine.logits[:B]) for _ in range(engine.T)]
    dist.all_gather(parts, engine.logits[:B].contiguous())
    return torch.cat(parts, dim=1).float()


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    hd = int(sys.argv[1]) if len(sys.argv) > 1 else 64
    heads, kv_heads = (4, 2) if world <= 2 else (2 * world, world)     # every rank owns at least one KV head
    cfg = LlamaConfig(vocab_size=512, max_ctx=96, embed_dim=heads * hd, num_layers=2, num_heads=heads,
                      num_kv_heads=kv_heads, ffn_dim=512 if world <= 4 else 1024, rope_base=10000.0, tie_weights=False, seed=3, init_std=0.05)
    ref = Llama(cfg).to("cuda", torch.bfloat16)          # same seed -> same weights on every rank
    ref.eval()
    eng = TPLlamaEngine(cfg, max_batch=4, max_ctx=96, max_rows=4 * 40, full_model=ref)
    B, S, NEW = 4, 40, 6
    g = torch.Generator().manual_seed(11)
    prompts = torch.randint(0, cfg.vocab_size, (B, S), generator=g).cuda()

    def check(tokens_so_far, tag):
        with torch.no_grad():
            want = ref(tokens_so_far)[:, -1, :].float()
        got = full_logits(eng, B)
        err = (got - want).abs().max().item()
        scale = want.abs().max().item()
        assert err < 0.06 * scale + 0.02, f"{tag}: logits differ by {err} (scale {scale})"
        # the exchanged argmax equals the argmax of the gathered logits
        assert torch.equal(eng.tokens[:B], got.argmax(-1)), f"{tag}: argmax exchange differs"

    for use_graph in (False, True):
        eng.reset()
        first = eng.prefill(prompts, chunk=2)
        seq = torch.cat([prompts, first.view(B, 1)], 1)
        check(prompts, f"prefill(graph={use_graph})")
        for step in range(NEW):
            nxt = eng.decode_step(B, use_graph=use_graph).clone()
            check(seq, f"decode {step} (graph={use_graph})")
            seq = torch.cat([seq, nxt.view(B, 1)], 1)
        assert int(eng.pos.item()) == S + NEW and eng.seq_len == S + NEW
        if use_graph:
            assert torch.equal(seq, eager_seq), "graph replay and eager decode disagree"
        eager_seq = seq
    out = eng.generate(prompts, NEW + 1)
    assert torch.equal(out, eager_seq)
    torch.cuda.synchronize()
    _native.raise_on_device_error()
    # sequence-parallel prefill (row-sharded activations: reduce-scatter / all-gather GEMMs) against the whole model
    # and against the all-reduce schedule; the rows of the call split into whole 128-row tiles per rank
    B2, S2 = 2 * world, 64
    eng2 = TPLlamaEngine(cfg, max_batch=B2, max_ctx=96, max_rows=B2 * S2, full_model=ref)
    p2 = torch.randint(0, cfg.vocab_size, (B2, S2), generator=g).cuda()
    with torch.no_grad():
        want = ref(p2)[:, -1, :].float()
    firsts = {}
    for mode in ("sp", "ar", "sp"):
        eng2.reset()
        firsts[mode] = eng2.prefill(p2, mode=mode).clone()
        got = full_logits(eng2, B2)
        err = (got - want).abs().max().item()
        assert err < 0.06 * want.abs().max().item() + 0.02, f"prefill mode {mode}: logits differ by {err}"
    nxt = eng2.decode_step(B2, use_graph=False).clone()        # the caches the sp prefill filled serve decode
    with torch.no_grad():
        want2 = ref(torch.cat([p2, firsts["sp"].view(B2, 1)], 1))[:, -1, :].float()
    err = (full_logits(eng2, B2) - want2).abs().max().item()
    assert err < 0.06 * want2.abs().max().item() + 0.02, f"decode after sp prefill: logits differ by {err}"
    torch.cuda.synchronize()
    _native.raise_on_device_error()
    dist.barrier()
    if rank == 0:
        print(f"tp_llama_worker ok (hd={hd}, nvls={eng.comm.use_nvls})")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
