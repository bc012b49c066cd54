"""CPU oracle for the sile hot path -- test infrastructure only.

Only tests, the smoke check and the bench's CPU-baseline legs may import this
package; the product (``sile_b200``) never does.
"""
from .loader import Oracle, build, load  # noqa: F401
