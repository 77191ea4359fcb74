"""Parity oracle of the CVM operator path (test infrastructure, not product code).

`run_model` is the numpy restatement (cvm_oracle.py); `ref_lib` drives the reference's own CPU
runtime when oracle/_ref/ has been built.  Importers: tests/, __graft_entry__.smoke(), and the CPU
baseline legs of bench.py.
"""
from . import cvm_oracle, ref_lib  # noqa: F401
from .cvm_oracle import Interpreter, run_model  # noqa: F401
