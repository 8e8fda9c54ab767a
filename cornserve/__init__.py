"""cornserve: a Blackwell-native any-to-any multimodal serving framework.

Layout:
  task/, app/, tasklib/        programming model (Task / UnitTask / Stream / DataForward, built-in tasks)
  services/                    gateway, task dispatcher, resource manager, task manager, registry, sidecar
  sidecar/                     tensor-forwarding client API
  executors/                   Eric (encoders), Geri (generators), LLM executor, monolithic baseline executor
  models/                      model definitions built on ``ops``
  ops/                         ctypes bindings of the sm_100a kernel library (``csrc/``) + fp32 references
  parallel/                    process groups, peer-memory fabric, fused compute+collective kernels
  utils/                       weight loading, logging, tracing, misc
"""

__version__ = "0.1.0"
