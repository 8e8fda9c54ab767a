"""Host-side logic of the parallel paths with two gloo ranks on the CPU: sequence-parallel diffusion transformer,
tensor-parallel vision tower and tensor-parallel decoder, each against the single-process model."""

import os
import subprocess
import sys

from cornserve.services.process import free_port


def test_parallel_models_two_gloo_ranks():
    script = os.path.join(os.path.dirname(__file__), "multiproc_cpu.py")
    port = str(free_port())
    env = dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="")
    procs = [subprocess.Popen([sys.executable, script, str(r), "2", port], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True, env=env) for r in range(2)]
    outs = [p.communicate(timeout=900)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs) and "MULTIPROC_CPU_OK" in outs[0], "\n".join(o[-3000:] for o in outs)
