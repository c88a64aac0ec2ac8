"""Load test against a running move server: python src/server/stress-test.py <port>"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from allie_b200.serve.stress_test import main  # noqa: E402

if __name__ == "__main__":
    main()
