//! Safe layer over the raw bindings, shaped for the three call sites in ruai's CUDA backend
//! (`CudaBackend::matmul_int8`, `dequant_int4`, `matmul_int4`; src/nn/backend/cuda.rs:788-833) and for
//! `Linear` (src/nn/modules/layers.rs:24-41, 169-190), which keeps the repacked weight next to its
//! `int8` / `int4` tensors so the repack happens once per layer, not once per call.
//!
//! Never compiled here (no Rust toolchain where the library is built); kept in step with the header by
//! tests/test_rust_shim.py.  Error behaviour follows the reference: a failure is a panic with the
//! library's message (cuda.rs:256, ops.rs:694-699).
use std::collections::HashMap;
use std::ffi::CStr;
use std::os::raw::{c_int, c_void};
use std::sync::{Arc, Mutex, OnceLock};

use crate::*;

/// One library context per device ordinal, like the leaked `CudaBackend` per ordinal (cuda.rs:82-86).
pub struct Ctx(pub *mut ruai_ctx);
unsafe impl Send for Ctx {}
unsafe impl Sync for Ctx {}

fn check(ctx: *const ruai_ctx, rc: c_int, what: &str) {
    if rc != RUAI_OK {
        let msg = unsafe { CStr::from_ptr(ruai_last_error(ctx)) }.to_string_lossy().into_owned();
        panic!("{what}: {msg}");
    }
}

/// The context of `ordinal`, created on first use on the backend's own stream (`cu_stream` is the
/// `CUstream` of `CudaBackend::stream`, so library work is ordered with the backend's kernels).
pub fn ctx_for(ordinal: usize, cu_stream: *mut c_void) -> &'static Ctx {
    static ALL: OnceLock<Mutex<HashMap<usize, &'static Ctx>>> = OnceLock::new();
    let mut all = ALL.get_or_init(|| Mutex::new(HashMap::new())).lock().unwrap();
    *all.entry(ordinal).or_insert_with(|| {
        let mut c: *mut ruai_ctx = std::ptr::null_mut();
        let rc = unsafe { ruai_ctx_create(ordinal as c_int, cu_stream, &mut c) };
        check(std::ptr::null(), rc, "ruai_ctx_create");
        Box::leak(Box::new(Ctx(c)))
    })
}

/// A repacked weight; freed with the `Linear` that owns it.
pub struct QWeight {
    ptr: *mut ruai_qweight,
}
unsafe impl Send for QWeight {}
unsafe impl Sync for QWeight {}

impl QWeight {
    /// From the device buffers of `Linear::int8`: `q` `[k, n]` I8, `scale` `[n]` F32 (layers.rs:34-35).
    pub fn int8(ctx: &Ctx, q_dev: u64, scale_dev: u64, k: usize, n: usize) -> Arc<QWeight> {
        let mut w = std::ptr::null_mut();
        let rc = unsafe { ruai_repack_int8(ctx.0, q_dev as *const i8, scale_dev as *const f32, k as u32, n as u32, &mut w) };
        check(ctx.0, rc, "ruai_repack_int8");
        Arc::new(QWeight { ptr: w })
    }
    /// From `Linear::int4`: `q` `[k/2, n]` packed, `scale` `[k/group, n]` (layers.rs:37-38).
    pub fn int4(ctx: &Ctx, q_dev: u64, scale_dev: u64, k: usize, n: usize, group: usize) -> Arc<QWeight> {
        let mut w = std::ptr::null_mut();
        let rc = unsafe { ruai_repack_int4(ctx.0, q_dev as *const i8, scale_dev as *const f32, k as u32, n as u32, group as u32, &mut w) };
        check(ctx.0, rc, "ruai_repack_int4");
        Arc::new(QWeight { ptr: w })
    }
}

impl Drop for QWeight {
    fn drop(&mut self) {
        unsafe { ruai_qweight_free(self.ptr) };
    }
}

/// `DType` of the activations as the library numbers it.
pub fn dtype_code(is_f16: bool, is_bf16: bool) -> c_int {
    if is_f16 { RUAI_F16 } else if is_bf16 { RUAI_BF16 } else { RUAI_F32 }
}

/// Body of `CudaBackend::matmul_int8` / `matmul_int4` for every `m`: `x_dev` `[m, k]`, `out_dev` `[m, n]`
/// freshly allocated by the backend in x's dtype (cuda.rs:805, 828).  The reference's `m > 16` branch
/// (dequantize + cuBLAS, cuda.rs:790-796, 822-827) is not needed: the library picks the kernel by `m`.
pub fn matmul_q(ctx: &Ctx, x_dtype: c_int, x_dev: u64, w: &QWeight, out_dev: u64, m: usize) {
    let rc = unsafe { ruai_matmul_q(ctx.0, x_dtype, x_dev as *const c_void, w.ptr, std::ptr::null(), out_dev as *mut c_void, m as u32) };
    check(ctx.0, rc, "ruai_matmul_q");
}

/// Body of `CudaBackend::dequant_int4` (cuda.rs:812-818): exact f32 `[k, n]` into `out_dev`.
pub fn dequant_int4(ctx: &Ctx, q_dev: u64, scale_dev: u64, k: usize, n: usize, group: usize, out_dev: u64) {
    let rc = unsafe { ruai_dequant_int4_ref(ctx.0, q_dev as *const i8, scale_dev as *const f32, k as u32, n as u32, group as u32, out_dev as *mut f32) };
    check(ctx.0, rc, "ruai_dequant_int4_ref");
}

/// Cache for callers that only have the `Storage` pointers (the `Backend` trait passes `&Storage`, not the
/// `Linear`): keyed by the device addresses of `q` and `scales`, which are immutable after creation
/// (backend/mod.rs:184-186).  `Linear::drop` (added by the patch) calls `forget`.
pub struct QWeightCache {
    map: Mutex<HashMap<(u64, u64), Arc<QWeight>>>,
}

impl QWeightCache {
    pub fn global() -> &'static QWeightCache {
        static C: OnceLock<QWeightCache> = OnceLock::new();
        C.get_or_init(|| QWeightCache { map: Mutex::new(HashMap::new()) })
    }
    pub fn int8(&self, ctx: &Ctx, q_dev: u64, scale_dev: u64, k: usize, n: usize) -> Arc<QWeight> {
        self.map.lock().unwrap().entry((q_dev, scale_dev)).or_insert_with(|| QWeight::int8(ctx, q_dev, scale_dev, k, n)).clone()
    }
    pub fn int4(&self, ctx: &Ctx, q_dev: u64, scale_dev: u64, k: usize, n: usize, group: usize) -> Arc<QWeight> {
        self.map.lock().unwrap().entry((q_dev, scale_dev)).or_insert_with(|| QWeight::int4(ctx, q_dev, scale_dev, k, n, group)).clone()
    }
    pub fn forget(&self, q_dev: u64, scale_dev: u64) {
        self.map.lock().unwrap().remove(&(q_dev, scale_dev));
    }
}
