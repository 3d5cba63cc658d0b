"""Drop-in module name of the reference extension (setup.py:5-7 builds `ff_attention`):
`from ff_attention import FastForwardAttn` keeps working against the B200 engine."""
from fastforwardattention_b200 import _extension as _ext

FastForwardAttn = _ext().FastForwardAttn
launch_count = _ext().launch_count
