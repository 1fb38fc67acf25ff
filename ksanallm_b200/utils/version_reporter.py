"""Version reporting hook. The reference calls a no-op ``VersionReporter`` singleton when ``is_version_report`` is
set (src/ksana_llm/periphery/version_reporter.h, used from src/ksana_llm/service/inference_engine.cpp:171,396-397);
here the hook logs the package version once at start-up and nothing leaves the process."""
import logging

VERSION = "0.1.0"
_started = False


def init(enabled: bool = True) -> bool:
    global _started
    if enabled and not _started:
        logging.getLogger("ksanallm_b200").info("ksanallm_b200 %s starting", VERSION)
        _started = True
    return _started


def stop_reporting() -> None:
    global _started
    _started = False
