"""CPU restatement (test infrastructure, not a product path) of the token shift around the WKV
operator: jaxrwkv src/jaxrwkv/rwkv7.py:226-235 and :254 (time mixing), :192-197 (channel mixing)."""
import numpy as np


def token_shift(x, prev, mix, length, new_starts):
    """x (T,D), prev (D,), mix (M,D), length int, new_starts (T,) bool -> (mixed (M,T,D), x[length-1])."""
    x = np.asarray(x)
    sx = np.concatenate([np.asarray(prev)[None], x[:-1]], axis=0)          # rwkv7.py:226
    sx = np.where(np.asarray(new_starts, bool)[:, None], 0, sx)             # rwkv7.py:227
    sx = sx - x                                                             # rwkv7.py:228
    mixed = x[None] + sx[None] * np.asarray(mix)[:, None, :]                # rwkv7.py:230-235
    return mixed, x[int(length) - 1]                                        # rwkv7.py:254 (length 0 wraps)
