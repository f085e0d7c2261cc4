"""Cooperative (DiLoCo-style) training: checkpoint averaging, corpus shards, model presets, HTTP star / gossip modes
(reference: lib/core/coop/*.dart, bin/coop_*.dart).  Inside one box, synchronous data parallelism
(``parallel/dp.py``) replaces it; these modes remain for loosely coupled workers."""
from .param_avg import average_checkpoints, averageCheckpoints
from .shard import CharVocab, K_TOY_CORPUS, kToyCorpus, sample_window, sampleWindow, shard_slice, shardSlice
from .lm_factory import Arch, CoopLM, build_coop_lm, buildCoopLM, parse_arch, arch_to_string
from .http_coop import Coordinator, Worker, Peer, train_phase0, local_steps
