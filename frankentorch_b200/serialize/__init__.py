"""``frankentorch_b200.serialize``: checkpoint envelope + sidecar, FTSV state dicts, SafeTensors, ONNX."""
from .checkpoint import (CODE_NAME, CheckpointEnvelope, CheckpointMode, DecodeMode, DecodeProofArtifact, RepairSymbolRecord,
                         decode_envelope, decode_snapshot, encode_envelope, encode_snapshot, RaptorQSidecar, RepairSidecar, SerializeError, SnapshotEntry,
                         checkpoint_hash, decode_checkpoint, decode_with_sidecar, encode_checkpoint,
                         generate_raptorq_sidecar, generate_repair_sidecar, hash_bytes, normalize_entries,
                         repair_symbol_count, symbol_size_for)
from .state_dict import (TensorIOError, load_safetensors_from_bytes, load_tensor_file, save_linear_onnx,
                         save_safetensors_to_bytes, consolidate_shards, export_linear_onnx_to_bytes, load_safetensors,
                         load_safetensors_metadata, load_state_dict, load_state_dict_from_bytes, save_safetensors,
                         save_sharded, save_state_dict, state_dict_to_bytes)
