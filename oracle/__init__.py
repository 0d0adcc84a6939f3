"""TEST INFRASTRUCTURE ONLY: CPU checkers for the message-passing operators.

Two checkers with one Python surface:

* ``port``  - ``libjgoracle.so``, this repository's plain-C restatement of the
  reference operators (``port.c``);
* ``ref``   - ``_ref/libjgref.so``, the reference's own CPU operator bodies
  compiled unmodified from a reference checkout (``Makefile``), when that
  library has been built.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
package.  The product (``jittorgeometric_b200``) never does.
"""
from .oracle import *  # noqa: F401,F403
