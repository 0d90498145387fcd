"""Process start timestamp, taken at first import (MFU 'including init' uses it).

Reference: ``nestor/utils/timing.py`` (``PROCESS_START`` imported first by the CLI).
"""

import time

PROCESS_START = time.monotonic()
