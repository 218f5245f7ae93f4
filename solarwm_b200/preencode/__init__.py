"""Pre-encoded dataset contracts and shard writers."""
from .contracts import EncoderContract, TensorSpec, validate_encoded_tensors  # noqa: F401
from .shards import EncodedShardWriter, read_encoded_sample, write_encoded_index  # noqa: F401
