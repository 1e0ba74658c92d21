"""Planning package: profiles -> cost model -> scheduler -> execution plan -> pipeline.
Pure Python; runs without a GPU."""
from .profiles import (CompressMethodProfile, ComputeType, BUILTIN_PROFILES, register_profile, get_profile,
                       list_profiles)
from .context import WorkloadContext, HardwareProfile, GPUArch, detect_hardware, get_hardware_profile
from .cost_model import CostModel, CalibrationData, should_compress
from .execution import (ExecutionPlan, ExecutionStep, ExecutionTiming, ParallelismMode, ParallelismConfig,
                        ChunkingConfig, StepType, PipelineExecutor, StreamManager, get_stream_manager)
from .scheduler import AutoCompressScheduler, SchedulerConfig, auto_schedule, analyze_compression
from .kernels import (TileLangKernelGenerator, KernelConfig, get_kernel_generator, get_mlp_kernel,
                      get_sparse_gather_kernel, get_quantize_kernels)
from .integration import (CompressionConfig, AutoCompressManager, AsyncCompressionHandle,
                          AdaptiveCompressionWrapper, create_auto_compress_manager, wrap_compressor,
                          analyze_workload)
from .methods import (CompressionMethod, MLPCompressionMethod, KVPressMethod, QuantizationMethod, MethodRegistry,
                      get_method, list_methods)
from .pipeline import (PipelineStrategy, PipelineConfig, ComposedPipelineConfig, PipelineOrchestrator,
                       create_optimal_pipeline, analyze_all_methods)

__version__ = "0.1.0"
