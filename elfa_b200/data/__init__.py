"""Token datasets (binary format, synthetic generators), loaders, packing and the BPE tokenizer."""
from .dataset import BinaryDataset, DataLoader, DatasetBuilder, ShardWriter, SyntheticDataset, write_token_file, Batch  # noqa: F401
from .packing import pack_sequences, StreamingPacker  # noqa: F401
from .tokenizer import Tokenizer  # noqa: F401
