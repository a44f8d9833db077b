"""Checkpoint loading: SafeTensors, GGUF, .gllm, PyTorch .bin, ONNX; quantised-tensor pairing; hub resolution."""
from .loader import (GgufProvider, LoadedModel, Loader, LoaderConfig, ModelNotFound, SafeTensorsProvider, TensorProvider,
                     WeightFormat, detect_format)
