"""cornserve: a Blackwell-native any-to-any multimodal serving framework.

Layout:
  task/, app/                  programming model (Task / UnitTask / Stream / DataForward); built-in tasks: cornserve_tasklib
  services/                    gateway, task dispatcher, resource manager, task manager, registry, sidecar
  sidecar/                     tensor-forwarding client API
  task_executors/              Eric (encoders), Geri (generators), LLM executor, monolithic baseline executor
  models/                      model definitions built on ``ops``
  ops/                         ctypes bindings of the sm_100a kernel library (``csrc/``) + fp32 references
  parallel/                    process groups, peer-memory fabric, fused compute+collective kernels
  utils/                       weight loading, logging, tracing, misc
"""

__version__ = "0.1.0"


def _exit_with_parent() -> None:
    """``CORNSERVE_EXIT_WITH_PARENT=1``: leave when the process that started this one is gone.

    A deployment is a tree of processes (control plane -> executors and sidecars -> tensor-parallel ranks), each in a
    session of its own.  When whoever started the tree is killed outright, nothing tells it to shut down, and executors
    that keep a whole GPU's memory outlive the run that wanted them.  With the variable set (it is inherited down the
    tree) every process of the tree watches its parent and exits as soon as it has been re-parented."""
    import os
    import threading
    import time

    if os.environ.get("CORNSERVE_EXIT_WITH_PARENT") != "1":
        return
    parent = os.getppid()

    def watch() -> None:
        while True:
            time.sleep(1.0)
            if os.getppid() != parent:
                os._exit(113)

    threading.Thread(target=watch, name="exit-with-parent", daemon=True).start()


_exit_with_parent()
