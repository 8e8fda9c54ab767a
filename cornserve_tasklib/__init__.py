"""Built-in task library: unit tasks, composite tasks and their execution descriptors.

Importing this package registers every built-in task class and descriptor in the in-process registries
(the reference ships its task library as a separate package whose sources are uploaded at run time:
tasklib/cornserve_tasklib/; uploading user-written task modules is still supported through the
task registry)."""

from cornserve_tasklib.task_executors.descriptor import encoder as _d_encoder  # noqa: F401
from cornserve_tasklib.task_executors.descriptor import generator as _d_generator  # noqa: F401
from cornserve_tasklib.task_executors.descriptor import huggingface as _d_huggingface  # noqa: F401
from cornserve_tasklib.task_executors.descriptor import llm as _d_llm  # noqa: F401
from cornserve_tasklib.task_executors.descriptor import omni as _d_omni  # noqa: F401
from cornserve_tasklib.task.composite.llm import DisaggregatedMLLMTask, MLLMEmbeddingTask, MLLMTask  # noqa: F401
from cornserve_tasklib.task.composite.omni import OmniInput, OmniTask  # noqa: F401
from cornserve_tasklib.task.unit.encoder import DummyEncoderTask, EncoderInput, EncoderOutput, EncoderTask, Modality  # noqa: F401
from cornserve_tasklib.task.unit.generator import (AudioGeneratorInput, AudioGeneratorTask, ImageGeneratorInput,  # noqa: F401
                                  ImageGeneratorOutput, ImageGeneratorTask)
from cornserve_tasklib.task.unit.huggingface import HuggingFaceQwenImageTask, HuggingFaceQwenOmniTask  # noqa: F401
from cornserve_tasklib.task.unit.llm import (DecodeLLMUnitTask, LLMEmbeddingResponse, LLMEmbeddingUnitTask, LLMUnitTask,  # noqa: F401
                            OpenAIChatCompletionChunk, OpenAIChatCompletionRequest, PrefillLLMUnitTask)
from cornserve_tasklib.task.unit.omni import OmniTalkerEmbeddingTask, OmniTalkerVocoderTask  # noqa: F401
