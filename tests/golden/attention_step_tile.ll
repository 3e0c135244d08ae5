define void @entry(i64 %0, i64 %1, i64 %2, i64 %3, i64 %4, i64 %5) {

  call void @wafer_tx81_rdma(i64 %0, i64 0, i32 16384, i32 16384, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_memset(i64 81920, i32 -8388608, i32 64, i32 5, i32 0)
  call void @wafer_tx81_memset(i64 83200, i32 0, i32 64, i32 5, i32 0)
  call void @wafer_tx81_memset(i64 98304, i32 0, i32 4096, i32 5, i32 0)
  br label %7
7:
  %8 = phi i64 [ 0, %6 ], [ %13, %9 ]
  %cond = icmp ult i64 %8, 2
  br i1 %cond, label %9, label %14
9:
  %off = mul i64 %8, 16384
  %ksrc = add i64 %1, %off
  %vsrc = add i64 %2, %off
  call void @wafer_tx81_rdma(i64 %ksrc, i64 16384, i32 16384, i32 16384, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_rdma(i64 %vsrc, i64 32768, i32 16384, i32 16384, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_gemm_oriented(i64 16384, i64 0, i64 49152, i64 0, i32 64, i32 64, i32 64, i32 1, i32 5, i32 5, i32 13, i32 0, i32 1, i32 0)
  call void @wafer_tx81_elementwise_mul(i64 49152, i64 1040187392, i64 49152, i32 4096, i32 5, i32 0, i32 1, i32 0, i32 1)
  call void @wafer_tx81_reduce_max(i64 49152, i64 82176, i32 1, i32 1, i32 1, i32 64, i32 64, i32 5, i32 1)
  call void @wafer_tx81_elementwise_max(i64 81920, i64 82176, i64 82432, i32 64, i32 5, i32 0, i32 0, i32 0, i32 1)
  call void @wafer_tx81_elementwise_sub(i64 81920, i64 82432, i64 82688, i32 64, i32 5, i32 0, i32 0, i32 0, i32 1)
  call void @wafer_tx81_elementwise_exp(i64 82688, i64 82944, i32 64, i32 5, i32 1)
  call void @wafer_tx81_elementwise_mul(i64 83200, i64 82944, i64 83456, i32 64, i32 5, i32 0, i32 0, i32 0, i32 1)
  call void @wafer_tx81_elementwise_sub(i64 49152, i64 82432, i64 65536, i32 4096, i32 5, i32 64, i32 0, i32 0, i32 1)
  call void @wafer_tx81_elementwise_exp(i64 65536, i64 65536, i32 4096, i32 5, i32 1)
  call void @wafer_tx81_reduce_sum(i64 65536, i64 83712, i32 1, i32 1, i32 1, i32 64, i32 64, i32 5, i32 1)
  call void @wafer_tx81_elementwise_add(i64 83456, i64 83712, i64 83200, i32 64, i32 5, i32 0, i32 0, i32 0, i32 1)
  call void @wafer_tx81_elementwise_mul(i64 98304, i64 82944, i64 114688, i32 4096, i32 5, i32 64, i32 0, i32 0, i32 1)
  call void @wafer_tx81_gemm_oriented(i64 32768, i64 65536, i64 98304, i64 114688, i32 64, i32 64, i32 64, i32 1, i32 5, i32 5, i32 5, i32 1, i32 0, i32 0)
  call void @wafer_tx81_elementwise_max(i64 82432, i64 82432, i64 81920, i32 64, i32 5, i32 0, i32 0, i32 0, i32 1)
  %13 = add nuw i64 %8, 1
  br label %7
14:
  call void @wafer_tx81_elementwise_recip(i64 83200, i64 83968, i32 64, i32 5, i32 1)
  call void @wafer_tx81_elementwise_mul(i64 98304, i64 83968, i64 114688, i32 4096, i32 5, i32 64, i32 0, i32 0, i32 1)
  call void @wafer_tx81_wdma(i64 114688, i64 %3, i32 16384, i32 16384, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_wdma(i64 81920, i64 %4, i32 256, i32 256, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  call void @wafer_tx81_wdma(i64 83200, i64 %5, i32 256, i32 256, i32 0, i32 0, i32 0, i32 1, i32 1, i32 1, i32 5, i32 0)
  ret void

}
!wafer.target.tile_id = !{!2}
!wafer.target.entry_arguments = !{!10, !11, !12, !13, !14, !15}
!2 = !{i64 0}
!10 = !{i64 0, !"external-input", i64 0, !"", !"f32", !"tensor", i64 16384, i64 4096, !"read-only", i64 64, i64 64, i64 0}
!11 = !{i64 1, !"external-input", i64 1, !"", !"f32", !"tensor", i64 32768, i64 8192, !"read-only", i64 128, i64 64, i64 0}
!12 = !{i64 2, !"external-input", i64 2, !"", !"f32", !"tensor", i64 32768, i64 8192, !"read-only", i64 128, i64 64, i64 0}
!13 = !{i64 3, !"external-output", i64 0, !"", !"f32", !"tensor", i64 16384, i64 4096, !"write-only", i64 64, i64 64, i64 0}
!14 = !{i64 4, !"external-output", i64 1, !"", !"f32", !"tensor", i64 256, i64 64, !"write-only", i64 64, i64 0}
!15 = !{i64 5, !"external-output", i64 2, !"", !"f32", !"tensor", i64 256, i64 64, !"write-only", i64 64, i64 0}
