"""CPU oracle for the hot path. TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and bench.py's
cpu_baseline / --impl reference legs; the product package never imports it."""
from oracle.oracle import *  # noqa: F401,F403
