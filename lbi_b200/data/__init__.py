from .lm_data import build_byte_stream, sample_batch_stream, split_stream_train_val
from .token_shards import TokenShardCorpus, TokenShardInfo, corpus_numel, sample_batch_token_shards
from .train_data import SYNTHETIC_TASKS, build_synthetic_corpus, sample_batch

__all__ = [
    "build_byte_stream", "sample_batch_stream", "split_stream_train_val", "TokenShardCorpus", "TokenShardInfo",
    "corpus_numel", "sample_batch_token_shards", "SYNTHETIC_TASKS", "build_synthetic_corpus", "sample_batch",
]
