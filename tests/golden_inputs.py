"""Seeded small inputs shared by the fixture generator tests/golden/make_ref_kernel_golden.py and the tests that read
its output (one definition, so the two cannot drift apart)."""
import importlib.util
import os

_spec = importlib.util.spec_from_file_location(
    "make_ref_kernel_golden", os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "make_ref_kernel_golden.py"))
_mod = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mod)
QUANTIZE_CASES, ROUTING_CASES = _mod.QUANTIZE_CASES, _mod.ROUTING_CASES
quantize_case_input, routing_case_input = _mod.quantize_case_input, _mod.routing_case_input
ATTENTION_CASES, attention_case_input = _mod.ATTENTION_CASES, _mod.attention_case_input
