"""jetfire_b200: B200-native (sm_100a) decode hot path of JetFire.

``ops`` mirrors the reference's operator surface on top of the C ABI in
``include/jetfire_b200.h``; ``adapter`` mirrors the pieces of its vLLM adapter that sit
on the hot path.  Importing ``ops`` loads ``libjetfire_b200.so`` and fails loudly if it
is missing -- there is no CPU or eager fallback.
"""
__version__ = "0.1.0"
