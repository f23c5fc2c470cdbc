//! The process-global library context and the backend type.
use std::ffi::CStr;
use std::sync::OnceLock;

use serde::{Deserialize, Serialize};
use stwo::prover::backend::Backend;

use crate::ffi;

/// The backend type (`CudaBackend`'s counterpart, `prover/backend/cuda/backend.rs:18-21`).
#[derive(Copy, Clone, Debug, Default, Serialize, Deserialize)]
pub struct B200Backend;

impl Backend for B200Backend {}

struct Handle(*mut ffi::ZkbCtx);
// The library serialises nothing itself: one host thread drives a context at a time. The generic prover calls the
// batched trait methods (interpolate_columns, evaluate_polynomials) from one thread; the per-column defaults that fan
// out over rayon are overridden in poly.rs for exactly this reason.
unsafe impl Send for Handle {}
unsafe impl Sync for Handle {}

static CTX: OnceLock<Handle> = OnceLock::new();

/// Creates the context: `device` is the CUDA device, `max_log_size` the largest evaluation domain (trace log size plus
/// blow-up) any later call will use. Call once before the first operator; later calls are ignored.
pub fn init(device: i32, max_log_size: u32) {
    CTX.get_or_init(|| {
        let mut p: *mut ffi::ZkbCtx = std::ptr::null_mut();
        let rc = unsafe { ffi::zkb_init(device, max_log_size as i32, &mut p) };
        assert!(rc == 0 && !p.is_null(), "zkb_init({device}, {max_log_size}) failed with status {rc}");
        Handle(p)
    });
}

/// The context; device 0 and 2^24 points unless `init` ran first.
pub(crate) fn ctx() -> *mut ffi::ZkbCtx {
    if CTX.get().is_none() {
        init(0, 24);
    }
    CTX.get().unwrap().0
}

/// Panics with the library's message on a non-zero status.
#[track_caller]
pub(crate) fn check(rc: i32) {
    if rc != 0 {
        let msg = unsafe { CStr::from_ptr(ffi::zkb_last_error(ctx())) }.to_string_lossy().into_owned();
        panic!("zkb200: status {rc}: {msg}");
    }
}
