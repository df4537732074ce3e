from .evaluator import Evaluator, Generator, benchmark_throughput, sample_top_p  # noqa: F401
from .harness import EvalHarness, lcs_length, rouge_l, rouge_n  # noqa: F401
from .needle import NeedleCase, depth_accuracy, generate_needle_case, generate_multi_needle  # noqa: F401
from .summary import SummaryCase, generate_summary_case, score_summary  # noqa: F401
