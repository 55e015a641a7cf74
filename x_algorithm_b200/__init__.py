"""B200-native Phoenix inference engine: ranking forward (multi-hash gather-sum -> transformer with
candidate-isolation attention -> heads -> weighted blend) and two-tower retrieval top-k, hand-written
CUDA for sm_100a behind a C ABI.  Importing the package loads the native library; there is no
fallback path."""
from ._lib import PhoenixError, LIB_PATH  # noqa: F401  (raises ImportError when the .so is missing)
from .config import PhoenixConfig, HashFamilySpec  # noqa: F401
from .engine import PhoenixEngine, RankInputs, RankOutputs  # noqa: F401
from .value_model import ValueModelWeights, blend_spec_from_weights, HEAD_NAMES_19  # noqa: F401
from .plugin import PhoenixScorer, PhoenixSource, ValueModelScorer, Candidate, Query  # noqa: F401
from .retrieval import CorpusShard  # noqa: F401
