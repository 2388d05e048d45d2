"""B200-native inference engine for the Qwen3 dense decoder of DavidAkinpelu/llm-pipeline, and for the Zupilorn hybrid
decoder (recurrent and latent-attention mixers, dense and routed-expert feed-forwards) and the Razelorn decoder (differential
attention beside its feed-forward on one layer norm, layers that share tensors) on the same parts and engine.

Sub-packages: ``config`` (typed configurations, architecture registry), ``weights`` (safetensors
loading, random model folders), ``parts`` (norm, position encoding, mixer, feed-forward, block),
``models`` (architectures assembled from parts), ``cache`` (paged keys/values, state slots),
``engine`` (step function, scheduler, generation), ``sampling``, ``ops`` (bindings of the CUDA
library built from ``csrc``).
"""

__version__ = "0.1.0"
