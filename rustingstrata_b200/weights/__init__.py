from .safetensors_io import (SafetensorsError, SafetensorsWriter, TensorEntry, TensorFileReader, read_header,
                             index_model_dir, f32_to_bf16_bits, bf16_bits_to_f32)
from .loader import WeightsError, load_checkpoint, match_names
from .random_init import write_random_model, draw_tensor
