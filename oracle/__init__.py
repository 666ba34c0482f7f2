"""TEST INFRASTRUCTURE: CPU oracle of the reference's hot path. Imported only by tests, smoke() and bench.py's CPU legs."""
