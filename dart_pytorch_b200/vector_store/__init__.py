"""Approximate-nearest-neighbour toolkit (reference: lib/core/vector_store/*.dart): exact, IVF, PQ, HNSW, LSH, scalar
quantised and binary indexes, transforms, shards / replicas, factory strings, conversions, benchmark + auto-tune,
``FAISDART`` persistence and FAISS binary interop, and a GPU brute-force index on the framework's GEMM."""
from .base import (Index, Metric, RangeSearchResult, SearchResult, TopK, as_rows, dot, l2sq, to_float32_rows)
from .flat import GPU_INDEX_FLAT_MIN_DOT, GpuIndexFlat, IndexFlat, IndexFlatIP, IndexFlatL2, Kmeans, KmeansResult
from .quantized import IndexIVFFlat, IndexIVFPQ, IndexPQ, IndexScalarQuantizer, ProductQuantizer
from .hnsw import IndexHNSW
from .composite import (IndexBinary, IndexBinaryFlat, IndexBinaryIVF, IndexIDMap, IndexLSH, IndexPreTransform,
                        IndexRefineFlat, IndexReplicas, IndexShards, L2NormTransform, PCATransform,
                        RandomRotationTransform, VectorTransform, hamming_distance, hammingDistance, jacobi_eigh,
                        popcount8_table)
from .tools import (BenchOptions, BenchResult, OperatingPoint, OperatingPoints, TuneMResult, auto_tune_ef_search,
                    auto_tune_m, auto_tune_m_from_flat, auto_tune_nprobe, autoTuneEfSearch, autoTuneM, autoTuneMFromFlat,
                    autoTuneNprobe, bench_index,
                    bench_index_sweep, benchIndex, benchIndexSweep, flat_to_hnsw, flat_to_ivf_flat, flat_to_ivf_pq,
                    flatToHnsw, flatToIvfFlat, flatToIvfPq, format_bench_table, formatBenchTable, index_factory,
                    indexFactory, pareto_frontier, paretoFrontier, recall_at_k, reconstruct_all, reconstructAll,
                    to_bench_csv, to_bench_markdown, toBenchCsv, toBenchMarkdown, wrap_with_refine, wrapWithRefine)
from .index_io import (IndexKind, read_binary_index, read_binary_index_bytes, read_index, read_index_bytes,
                       readBinaryIndex, readIndex, write_binary_index, write_index, write_index_bytes,
                       writeBinaryIndex, writeIndex)
from .faiss_io import (FaissFourcc, faiss_describe, faiss_strip, read_faiss_binary_index,
                       read_faiss_binary_index_bytes, read_faiss_index, read_faiss_index_bytes, readFaissBinaryIndex,
                       readFaissIndex, write_faiss_binary_index, write_faiss_binary_index_bytes, write_faiss_index,
                       write_faiss_index_bytes, writeFaissBinaryIndex, writeFaissIndex, saveFaissIndex, loadFaissIndex,
                       saveFaissBinaryIndex, loadFaissBinaryIndex, writeFaissIndexToBytes, readFaissIndexFromBytes,
                       writeFaissBinaryIndexToBytes, readFaissBinaryIndexFromBytes)
from .faiss_tuned import (FaissIndexInfo, FaissIndexKind, TuningMetadata, apply_tuning_to_index, applyTuningToIndex,
                          is_tuned_faiss_blob, isTunedFaissBlob, load_tuned_faiss_index, loadTunedFaissIndex,
                          probe_faiss_index, probe_faiss_index_file, probeFaissIndex, probeFaissIndexFile,
                          read_tuned_faiss_index_bytes, readTunedFaissIndexFromBytes, save_tuned_faiss_index,
                          saveTunedFaissIndex, strip_tuning_wrapper, strip_tuning_wrapper_file, stripTuningWrapper,
                          stripTuningWrapperFile, write_tuned_faiss_index_bytes, writeTunedFaissIndexToBytes)
