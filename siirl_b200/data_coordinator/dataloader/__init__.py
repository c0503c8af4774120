from .data_loader_node import DataLoaderNode  # noqa: F401
from .partitioned_dataset import PartitionedRLHFDataset, collate_fn, left_pad  # noqa: F401
from .tokenizer import SyntheticTokenizer, load_tokenizer  # noqa: F401
