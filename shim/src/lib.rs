//! `B200Backend`: the reference's operator traits over `libzkb200.so`.
//!
//! The traits have no context argument (`prover/backend/mod.rs:20-37`), so one process-global library context sits
//! behind a `OnceLock` (`ctx.rs`), as the reference's CUDA backend keeps its device pool global. Every trait method is
//! pointer plumbing around one `zkb_*` call; a non-zero status panics with the library's message (the traits are
//! infallible and the existing backends `assert!`).
//!
//! Selecting it in the prover: `#[cfg(feature = "b200")] pub type PcsB = zkb200_backend::B200Backend;` beside the two
//! existing arms at `prover/src/common.rs:163-166`.
pub mod ffi;

mod accumulation;
mod column;
mod ctx;
mod fri;
mod gkr;
mod grind;
mod merkle;
mod poly;
mod quotients;

pub use column::{B200BaseColumn, B200HashColumn, B200SecureColumn};
pub use ctx::{init, B200Backend};
