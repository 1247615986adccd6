"""``frankentorch_b200.nn``: module system and layers on the DAC tape (mirror of ft-nn)."""
from .layers import *  # noqa: F401,F403
from .layers import _param  # noqa: F401
from .enums import (CTCReduction, DistanceKind, EmbeddingBagMode, PaddingMode, Reduction, TransformerActivation,  # noqa: F401
                    UpsampleMode)
from .module import (LoadStateDictReport, Module, ModuleDict, ModuleError, ModuleList, ModuleRegistrationError, StateDictError, ParameterDict, ParameterList,
                     Sequential, StateDict, clip_grad_norm_, clip_grad_value_, module_load_state_dict,
                     module_state_dict, named_buffers, named_modules, named_parameters, parameters_to_vector,
                     vector_to_parameters)
from .transformer import *  # noqa: F401,F403
from .extra import (AdaptiveLogSoftmaxWithLoss, FractionalMaxPool2d, FractionalMaxPool3d, GRUOutput,  # noqa: F401
                    LazyConv1d, LazyConv2d, LazyConv3d, LPPool3d, LSTMOutput, MaxPool2dWithIndices, MaxUnpool1d,
                    MaxUnpool2d, MaxUnpool3d, MultiLabelMarginLoss, MultiLabelSoftMarginLoss, RNNConfig, RNNOutput,
                    TripletMarginWithDistanceLoss, Upsample, Upsample1d, Upsample2d, Upsample3d,
                    UpsamplingBilinear2d, UpsamplingNearest2d)
from .utils import (MinMaxObserver, PackedSequence, QParams, QuantizedLinear, QuantizedLinearQParams,
                    QuantizedLinearWeightStorage, QuantizedStorageDType, SpectralNorm, WeightNorm, dequantize,
                    pack_padded_sequence, pack_sequence, pad_packed_sequence, pad_sequence, quantize_per_tensor,
                    spectral_norm, weight_norm, weight_norm_decompose, weight_norm_reconstruct)
from . import builders  # noqa: F401,E402  (reference-style constructors and named forwards, attached to the classes above)
from .utils import qint8_range, quint8_range  # noqa: F401,E402
