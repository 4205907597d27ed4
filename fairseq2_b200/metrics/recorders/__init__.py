from fairseq2_b200.metrics.recorders.recorder import (CompositeMetricRecorder, JsonlMetricRecorder,
                                                      LogMetricRecorder, MetricDescriptor, MetricRecorder,
                                                      NoopMetricRecorder, TensorBoardRecorder, WandbRecorder,
                                                      format_metric_value, get_metric_descriptor,
                                                      register_metric_descriptor)
