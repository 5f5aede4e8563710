"""swlm-b200: host-side mirror of swift-lm's decode/prefill interface over libswlm_cuda.so.

The directory name carries a hyphen, so import it through ``load_package()`` of the
repository-root helpers (tests/conftest.py, bench.py) or with importlib; inside the package
relative imports are used throughout.

Nothing here computes: every numeric path goes through the C ABI declared in include/swlm.h,
and loading fails loudly when the CUDA library has not been built.
"""
from .lib import Library, SwlmError, load_library  # noqa: F401
from .formats import (  # noqa: F401
    AffineQ4Group64Format,
    AffineQ4Group128Format,
    KVCacheSpecification,
    bf16_to_f32,
    f32_to_bf16,
    pack_mlx_q4,
)
from .plan import (  # noqa: F401
    BuffersDesc,
    DispatchPlanBuilder,
    ModelConfig,
    Step,
    llama3_8b_config,
    lfm2_like_config,
)
from .model import InferenceModel, WeightStore, bundle_tensors, load_model, load_model_from_staf  # noqa: F401
from . import bundle, formats, plan, staf, tp  # noqa: F401
from .bundle import load_bundle, prepare_bundle  # noqa: F401
from .synth import synth_model_weights, synth_q4  # noqa: F401
