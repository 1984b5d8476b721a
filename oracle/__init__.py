"""CPU oracle for the b200 backend: a restatement of the reference's cc (C)
backend code generation.  TEST INFRASTRUCTURE ONLY — imported by tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline leg, never by the shipped
package."""
