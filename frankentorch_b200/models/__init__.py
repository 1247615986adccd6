
from .encoder import EncoderGpu, EncoderLayerWeights  # noqa: E402,F401
