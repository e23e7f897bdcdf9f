"""quant_format_list: prints the format table (tools/format_list.cpp)."""
import sys


def main(argv=None):
    from ..quant.planner import FormatRegistry
    sys.stdout.write(FormatRegistry.get_format_table())
    return 0


if __name__ == "__main__":
    sys.exit(main())
