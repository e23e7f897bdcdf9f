"""gle_report <log.jsonl>: event counts, verdict tallies and hash-chain verification (tools/gle_report.cpp)."""
import sys


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        print("Usage: gle_report <telemetry.jsonl>")
        return 1
    from ..utils import gle
    sys.stdout.write(gle.report(argv[0]))
    return 0 if gle.TelemetryReader(argv[0]).report().chain_valid else 3


if __name__ == "__main__":
    sys.exit(main())
