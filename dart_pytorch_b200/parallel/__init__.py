"""Multi-GPU parallelism over NVLink 5 / NVSwitch: data parallel (fused all-reduce + clip partials), tensor parallel,
expert parallel.  ``torch.distributed`` (NCCL) provides rendezvous, symmetric-memory allocation and the baseline paths;
the product paths are this package's own kernels issuing peer / multimem traffic."""
