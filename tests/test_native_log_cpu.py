"""Native runtime logging: level control, the error record of a failing entry point, forwarding into `logging`."""
import logging

from ooverlap_b200 import _lib
from ooverlap_b200.utils import logging as oob_logging


def test_levels_and_forwarding(caplog):
    lib = _lib.lib()
    before = lib.oob_get_log_level()
    try:
        assert lib.oob_set_log_level(9) == _lib.ERR_INVALID
        oob_logging.set_native_log_level("debug")
        assert lib.oob_get_log_level() == _lib.LOG_DEBUG
        oob_logging.forward_native_logs(True)
        oob_logging.logger.setLevel(logging.DEBUG)
        oob_logging.logger.propagate = True
        with caplog.at_level(logging.DEBUG, logger="ooverlap_b200"):
            lib.oob_log_message(_lib.LOG_WARN, b"hello from the test")
            assert lib.oob_policy_load(b"/nonexistent/policy.json") != 0      # a failing entry point logs its message
            oob_logging.set_native_log_level("error")
            lib.oob_log_message(_lib.LOG_INFO, b"this one is filtered out")
        text = caplog.text
        assert "native: hello from the test" in text
        assert "native: error" in text and "policy.json" in text
        assert "filtered out" not in text
    finally:
        oob_logging.forward_native_logs(False)
        oob_logging.logger.propagate = False
        oob_logging.setup()
        lib.oob_set_log_level(before)
        lib.oob_policy_load(b"")
