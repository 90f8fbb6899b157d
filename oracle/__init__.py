"""TEST INFRASTRUCTURE: CPU oracle for the CompressGNN hot path (see ``oracle.py``).

Nothing in the product package may import from here.
"""
