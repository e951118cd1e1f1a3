from .decoder import DecoderModel, expected_tensors  # noqa: F401
