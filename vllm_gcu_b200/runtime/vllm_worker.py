"""Worker class that vLLM's executors start on every GPU when the platform plugin is active
(``parallel_config.worker_cls``, set by ``B200Platform.check_and_update_config``; the
reference points it at its own worker, vllm_gcu/gcu.py:192-209 and
vllm_gcu/worker/worker_v1.py:236).  It is vLLM's GPU worker plus the start-up duties of this
package: the native library must load (a missing ``_b200.so`` on a GPU box is an error, not
a silent fallback) and the layer kernels are registered before the model is built."""
from __future__ import annotations

from vllm.v1.worker.gpu_worker import Worker


class B200Worker(Worker):
    def init_device(self):
        from ..ops import _native
        from . import vllm_ops
        if _native.lib() is None:
            raise RuntimeError("vllm_gcu_b200: the native library is not built")
        vllm_ops.register_ops()
        return super().init_device()

    def native_launch_count(self) -> int:
        """Kernels of this package launched by this worker process so far."""
        from ..ops import _native
        return int(_native.launch_count)
