"""Runnable programs: training demos, inference runners with HTTP serving, the RAG chat server, cooperative-training
roles and vector-store tools (reference: bin/*.dart).  ``python -m dart_pytorch_b200.apps --help`` lists them."""
from .util import (generate_text, get_window, last_row_logits, load_corpus, param_scalar_count, sample_from_logits)
from .servers import (GenerationService, LlamaChat, RagChatService, center_and_normalize, chunk_spans,
                      llama3_chat_prompt, load_hf_model, mean_vector)
