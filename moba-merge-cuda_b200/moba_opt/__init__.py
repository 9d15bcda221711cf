"""moba_opt: B200-native MoBA sparse attention behind the reference's public names
(src/moba_opt/__init__.py:3-7): the implementation registry, `opt_gqa_cuda` prefill with autograd,
and the KV caches with prepared decode."""
from . import api  # noqa: F401
from . import grouped_attention  # noqa: F401  (registers "opt_gqa_cuda")
from .api import available_impls, register, run_impl  # noqa: F401
from .kv_cache import AppendResult, ContiguousKVCache, DecodeResult, PagedKVCache  # noqa: F401,E402
from .prepared_decode import PreparedDecode  # noqa: F401,E402
